// A float32 residual stream whose layers are joined over depth: behind layer i the stream becomes a
// learnt weighted sum of the embedding output X_0 and of every layer result X_1 .. X_(i+1),
//
//     x <- sum_j a_i[j] X_j,        X_(i+1) = x + m f(norm(x)) (+ m g(norm(.)) for a second sublayer),
//
// with pre-norm sublayers whose outputs enter the stream times a constant m.  The results live in one
// buffer [levels, tokens, hidden] of floats.  Everything that touches a row between two sublayers is
// ONE kernel, as the residual sum and the norm after it are one kernel elsewhere in this library:
//
//     v = base + m y                      y: the output of the sublayer before (working type), or none
//     mix given:   X_(levels-1) = v  is filed,  x = sum_(j < levels) mix[j] X_j      (a layer's end)
//     otherwise:   x = v                                                              (inside a layer)
//     x is written to `dst` (where the next sublayer's output will add onto it), and
//     out = norm(x) * gain in the working type, for the sublayer that follows.
//
// With `rows` only those rows are computed and nothing but `out` is written: the model's end.
// The norm is either a layer norm without bias ((x - mean) / sqrt(mean((x - mean)^2) + eps)) or a
// root-mean-square norm (x / sqrt(mean(x^2) + eps)); sums, means and the row are float.
#include "common.cuh"

#define DEPTH_NORM_RMS 0
#define DEPTH_NORM_LAYER 1

template <typename T>
__global__ void depth_step_kernel(const float* __restrict__ base, const T* __restrict__ y, float mult,
                                  float* __restrict__ history, size_t level_stride, const float* __restrict__ mix,
                                  int levels, float* __restrict__ dst, const float* __restrict__ gain,
                                  T* __restrict__ out, const int* __restrict__ rows, int hidden, float eps,
                                  int norm_kind) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(base);
  SB_BEHIND_WAIT(y);
  SB_BEHIND_WAIT(history);
  SB_BEHIND_WAIT(rows);
  const int out_row = blockIdx.x;
  const int in_row = rows ? rows[out_row] : out_row;
  const size_t at = (size_t)in_row * hidden;
  float sum = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float v = base[at + c];
    if (y) v += mult * to_f<T>(y[at + c]);
    if (mix) {
      if (!rows) history[(size_t)(levels - 1) * level_stride + at + c] = v;
      float x = mix[levels - 1] * v;
      for (int j = 0; j < levels - 1; ++j) x += mix[j] * history[(size_t)j * level_stride + at + c];
      v = x;
    }
    if (dst && !rows) dst[at + c] = v;
    row[c] = v;
    sum += norm_kind == DEPTH_NORM_LAYER ? v : v * v;
  }
  if (!out) return;
  sum = block_sum(sum, scratch);
  float mean = 0.f, inv;
  if (norm_kind == DEPTH_NORM_LAYER) {
    mean = sum / (float)hidden;
    float sq = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
      const float d = row[c] - mean;
      sq += d * d;
    }
    sq = block_sum(sq, scratch);
    inv = 1.f / sqrtf(sq / (float)hidden + eps);
  } else {
    inv = 1.f / sqrtf(sum / (float)hidden + eps);
  }
  T* o = out + (size_t)out_row * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) o[c] = from_f<T>((row[c] - mean) * inv * gain[c]);
}

// logits <- cap * tanh(logits / cap), in place, float.
__global__ void softcap_kernel(float* __restrict__ x, size_t total, float cap) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(x);
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) x[i] = cap * tanhf(x[i] / cap);
}

extern "C" {

// base: float [*, hidden] (the rows v starts from).  y: null or [*, hidden] of the working type.  history:
// float [levels, n_tokens, hidden] with level_stride = n_tokens * hidden, or null when mix is null.  mix:
// null or float [levels].  dst: null or float [*, hidden].  gain / out: null (only the sums), or float
// [hidden] and [n_rows, hidden] of the working type.  rows: null (every row) or int [n_rows].
int sb_depth_step(int dtype, const float* base, const void* y, float mult, float* history, long long level_stride,
                  const float* mix, int levels, float* dst, const float* gain, void* out, const int* rows,
                  int n_rows, int hidden, float eps, int norm_kind, cudaStream_t s) {
  if (n_rows == 0) return 0;
  if ((out && !gain) || (mix && (!history || levels < 1))) return -2;
  if (norm_kind != DEPTH_NORM_RMS && norm_kind != DEPTH_NORM_LAYER) return -2;
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const int threads = hidden >= 2048 ? 512 : hidden >= 512 ? 256 : 128;
  if (dtype == 0) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(depth_step_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(depth_step_kernel<float>, dim3(n_rows), dim3(threads), smem, s, base, (const float*)y, mult,
                            history, (size_t)level_stride, mix, levels, dst, gain, (float*)out, rows, hidden, eps,
                            norm_kind);
  }
  if (smem > 48 * 1024) cudaFuncSetAttribute(depth_step_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  return launch_dependent(depth_step_kernel<bf16>, dim3(n_rows), dim3(threads), smem, s, base, (const bf16*)y, mult,
                          history, (size_t)level_stride, mix, levels, dst, gain, (bf16*)out, rows, hidden, eps,
                          norm_kind);
}

int sb_softcap(float* x, long long total, float cap, cudaStream_t s) {
  if (total <= 0) return 0;
  if (!(cap > 0.f)) return -2;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return launch_dependent(softcap_kernel, dim3((int)blocks), dim3(256), 0, s, x, (size_t)total, cap);
}

}  // extern "C"
