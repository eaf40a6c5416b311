// Per-channel mechanisms of recurrent mixers, over the packed tokens of a step and the per-sequence state in
// the cache's slots:
//
//   short_conv   a causal convolution over time, one filter of K taps per channel:
//                    y[t, c] = act(b[c] + sum_j taps[c, K - 1 - j] * (x[t - j, c] + b_in[c]))
//                with zeros in front of the sequence.  The last K - 1 inputs of every sequence live in its
//                slot (float, newest first), so a prompt, a later portion of it and a single token are the
//                same code: the first tokens of a portion see what the tokens before it left.
//   glru_scan    the real-gated linear recurrent unit, per channel:
//                    r = sigmoid(zr + br), i = sigmoid(zi + bi)            (gate logits from block-diagonal products)
//                    log a = -c * r * softplus(lam), S <- a S + sqrt(1 - a^2) * i * u,  out = S * gelu_tanh(y + by)
//                with S float in the slot, from zero for a new sequence, every token alike.
//
// Sums, the gates, the decay with its logarithm, the state and the activations are float whatever the working
// type T; inputs and outputs of the working type are rounded once, where they are stored.
//
// A long portion is cut into chunks of tokens that run as separate blocks.  short_conv: a chunk's first
// tokens read the inputs in front of it; only a sequence's first chunk reads the slot, and the same thread
// writes it at the end, so no block reads what another writes.  glru_scan: the recurrence is linear in S, so
// a warp a segment of tokens first forms its segment's (product of a, sum) pair from a zero state, the
// pairs are chained through shared memory, and each warp then walks its segment again from its true start.
// Decays travel as their complements 1 - a (products of them as -expm1 of the summed logarithms).
#include "common.cuh"

#define CONV_MAX_TAPS 8
#define CONV_CHUNK 32
#define CONV_BATCH 8      // tokens whose loads are in flight together

template <typename T>
__global__ void __launch_bounds__(128)
short_conv_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ taps, const float* __restrict__ bias,
                  const float* __restrict__ in_bias, T* __restrict__ y, int ldy, float* __restrict__ state,
                  long long slot_stride, const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                  const int* __restrict__ seq_q_len, int channels, int K, int act, int chunks) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(x);
  SB_BEHIND_WAIT(state);
  SB_BEHIND_WAIT(seq_slot);
  SB_BEHIND_WAIT(seq_q_start);
  SB_BEHIND_WAIT(seq_q_len);
  const int seq = blockIdx.x / chunks, chunk = blockIdx.x - seq * chunks;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int q_len = seq_q_len[seq];
  const int t0 = chunk * CONV_CHUNK;
  if (c >= channels || t0 >= q_len) return;
  const int q_start = seq_q_start[seq];
  float* st = state + (size_t)seq_slot[seq] * slot_stride + c;      // row j: the input j + 1 tokens back
  const float ib = in_bias ? in_bias[c] : 0.f;
  // tap[j] multiplies the input j + 1 tokens back; entries from K - 1 on are zero
  float tap[CONV_MAX_TAPS - 1], recent[CONV_MAX_TAPS - 1], old[CONV_MAX_TAPS - 1];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
    tap[j] = j < K - 1 ? taps[(size_t)c * K + (K - 2 - j)] : 0.f;
    float v = 0.f;
    if (j < K - 1) {
      const int t = t0 - 1 - j;
      v = t >= 0 ? to_f<T>(x[(size_t)(q_start + t) * ldx + c]) + ib : st[(size_t)(-t - 1) * channels];
    }
    recent[j] = old[j] = v;
  }
  const float now = taps[(size_t)c * K + K - 1], b = bias ? bias[c] : 0.f;
  const int t1 = min(t0 + CONV_CHUNK, q_len);
  for (int tb = t0; tb < t1; tb += CONV_BATCH) {
    float in[CONV_BATCH];
#pragma unroll
    for (int i = 0; i < CONV_BATCH; ++i)
      in[i] = tb + i < t1 ? to_f<T>(x[(size_t)(q_start + tb + i) * ldx + c]) + ib : 0.f;
#pragma unroll
    for (int i = 0; i < CONV_BATCH; ++i) {
      if (tb + i >= t1) break;
      const float v = in[i];
      float a = b + now * v;
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) a += tap[j] * recent[j];
#pragma unroll
      for (int j = CONV_MAX_TAPS - 2; j > 0; --j) recent[j] = recent[j - 1];
      recent[0] = v;
      if (act == 1) a = a / (1.f + expf(-a));
      y[(size_t)(q_start + tb + i) * ldy + c] = from_f<T>(a);
    }
  }
  if (chunk != 0) return;
  // what the sequence's next step will find in front of it: its last K - 1 inputs, those of earlier
  // steps (held in `old`, read before anything is written) where this step brought fewer
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
    if (j >= K - 1) break;
    const int t = q_len - 1 - j;
    float v = 0.f;
    if (t >= 0) {
      v = to_f<T>(x[(size_t)(q_start + t) * ldx + c]) + ib;
    } else {
#pragma unroll
      for (int o = 0; o < CONV_MAX_TAPS - 1; ++o)
        if (o == -t - 1) v = old[o];
    }
    st[(size_t)j * channels] = v;
  }
}

// ------------------------------------------------------------------------------------------ the gated unit

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

#define GLRU_BATCH 8      // tokens whose loads are in flight together

// One token of one channel: the decay's logarithm, its complement d = 1 - a and what enters the state, from its
// gate logits and its input.  A decay close to one is kept as its complement: rounding a itself to a float would
// lose up to 2^-24 / (1 - a) of the RATE of the decay, which is what a long memory is made of; S - d * S does not.
__device__ __forceinline__ void glru_terms(float zr, float zi, float u, float br, float bi, float rate, float& log_a,
                                           float& d, float& in) {
  const float r = 1.f / (1.f + expf(-(zr + br)));
  const float i = 1.f / (1.f + expf(-(zi + bi)));
  log_a = -rate * r;                                   // rate = c * softplus(lam)
  d = -expm1f(log_a);
  in = sqrtf(-expm1f(2.f * log_a)) * i * u;
}

// Block = 32 channels (lanes) x `segments` warps; warp w walks tokens [w * per, (w + 1) * per) of its
// sequence.  gates: float [blocks][n_tokens][2 * bs], a block's r logits then its i logits.
template <typename T>
__global__ void __launch_bounds__(1024)
glru_scan_kernel(const T* __restrict__ u, int ldu, const float* __restrict__ gates, int n_tokens, int bs,
                 const float* __restrict__ r_bias, const float* __restrict__ i_bias, const float* __restrict__ lam,
                 float decay_scale, const T* __restrict__ ybranch, int ldy, const float* __restrict__ y_bias,
                 T* __restrict__ out, float* __restrict__ state, long long slot_stride,
                 const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                 const int* __restrict__ seq_q_len, int channels) {
  __shared__ float carry_a[32][33], carry_s[32][33];
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(u);
  SB_BEHIND_WAIT(gates);
  SB_BEHIND_WAIT(ybranch);
  SB_BEHIND_WAIT(state);
  SB_BEHIND_WAIT(seq_slot);
  SB_BEHIND_WAIT(seq_q_start);
  SB_BEHIND_WAIT(seq_q_len);
  const int seq = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int c = blockIdx.y * 32 + lane;
  const bool real = c < channels;
  const int cc = real ? c : channels - 1;
  const int q_start = seq_q_start[seq], q_len = seq_q_len[seq];
  const int per = (q_len + warps - 1) / warps;
  const int t0 = min(warp * per, q_len), t1 = min(t0 + per, q_len);
  const int blk = cc / bs, o = cc - blk * bs;
  const float* zr = gates + (size_t)blk * n_tokens * 2 * bs + o;
  const float* zi = zr + bs;
  const float br = r_bias[cc], bi = i_bias[cc], rate = decay_scale * softplus_f(lam[cc]);
  const float yb = y_bias ? y_bias[cc] : 0.f;
  float* st = state + (size_t)seq_slot[seq] * slot_stride + cc;
  float S = 0.f;
  if (warps > 1) {
    // the segment from a zero state: S_end = A * S_start + B, with A kept as the sum of its logarithms
    float A = 0.f, B = 0.f;
    for (int tb = t0; tb < t1; tb += GLRU_BATCH) {
      float vr[GLRU_BATCH], vi[GLRU_BATCH], vu[GLRU_BATCH];
#pragma unroll
      for (int n = 0; n < GLRU_BATCH; ++n) {
        const size_t row = (size_t)(q_start + min(tb + n, t1 - 1));
        vr[n] = zr[row * 2 * bs];
        vi[n] = zi[row * 2 * bs];
        vu[n] = to_f<T>(u[row * ldu + cc]);
      }
#pragma unroll
      for (int n = 0; n < GLRU_BATCH; ++n) {
        if (tb + n >= t1) break;
        float log_a, d, in;
        glru_terms(vr[n], vi[n], vu[n], br, bi, rate, log_a, d, in);
        A += log_a;
        B = fmaf(-d, B, B) + in;
      }
    }
    carry_a[warp][lane] = -expm1f(A);
    carry_s[warp][lane] = B;
    __syncthreads();
    S = *st;
    for (int w = 0; w < warp; ++w) S = fmaf(-carry_a[w][lane], S, S) + carry_s[w][lane];
  } else {
    S = *st;
  }
  for (int tb = t0; tb < t1; tb += GLRU_BATCH) {
    float vr[GLRU_BATCH], vi[GLRU_BATCH], vu[GLRU_BATCH], vy[GLRU_BATCH];
#pragma unroll
    for (int n = 0; n < GLRU_BATCH; ++n) {
      const size_t row = (size_t)(q_start + min(tb + n, t1 - 1));
      vr[n] = zr[row * 2 * bs];
      vi[n] = zi[row * 2 * bs];
      vu[n] = to_f<T>(u[row * ldu + cc]);
      vy[n] = to_f<T>(ybranch[row * ldy + cc]);
    }
#pragma unroll
    for (int n = 0; n < GLRU_BATCH; ++n) {
      if (tb + n >= t1) break;
      float log_a, d, in;
      glru_terms(vr[n], vi[n], vu[n], br, bi, rate, log_a, d, in);
      S = fmaf(-d, S, S) + in;
      if (real) out[(size_t)(q_start + tb + n) * channels + c] = from_f<T>(S * gate_act(vy[n] + yb, SB_ACT_GELU_TANH));
    }
  }
  // the warp whose segment ends the sequence holds the state the next step starts from
  // (behind a barrier: every warp has read the old state by now)
  if (warps > 1) __syncthreads();
  if (real && t0 < t1 && t1 == q_len) *st = S;
}

extern "C" {

int sb_conv_max_taps() { return CONV_MAX_TAPS; }

// x: [n_tokens, ldx] (the channels start at the pointer), y: [n_tokens, ldy]; taps float [channels, K], bias and
// in_bias float [channels] or null; state: float, a slot's K - 1 rows of `channels` start at the pointer, slots
// slot_stride floats apart; act 0: none, 1: silu.  max_q_len: the most tokens a sequence brings.
int sb_short_conv(int dtype, const void* x, int ldx, const float* taps, const float* bias, const float* in_bias, void* y,
                  int ldy, float* state, long long slot_stride, const int* seq_slot, const int* seq_q_start,
                  const int* seq_q_len, int n_seqs, int max_q_len, int channels, int K, int act, cudaStream_t s) {
  if (n_seqs == 0 || channels == 0) return 0;
  if (K < 1 || K > CONV_MAX_TAPS || K - 1 > CONV_CHUNK || max_q_len < 1) return -2;
  const int chunks = (max_q_len + CONV_CHUNK - 1) / CONV_CHUNK;
  const dim3 grid(n_seqs * chunks, (channels + 127) / 128);
  if (dtype == 0)
    return launch_dependent(short_conv_kernel<float>, grid, dim3(128), 0, s, (const float*)x, ldx, taps, bias, in_bias,
                            (float*)y, ldy, state, slot_stride, seq_slot, seq_q_start, seq_q_len, channels, K, act, chunks);
  return launch_dependent(short_conv_kernel<bf16>, grid, dim3(128), 0, s, (const bf16*)x, ldx, taps, bias, in_bias,
                          (bf16*)y, ldy, state, slot_stride, seq_slot, seq_q_start, seq_q_len, channels, K, act, chunks);
}

// u: [n_tokens, ldu], ybranch: [n_tokens, ldy] (working type); gates: float [channels / bs][n_tokens][2 * bs];
// out: [n_tokens, channels]; state: float, a slot's `channels` entries start at the pointer.
int sb_glru_scan(int dtype, const void* u, int ldu, const float* gates, int n_tokens, int bs, const float* r_bias,
                 const float* i_bias, const float* lam, float decay_scale, const void* ybranch, int ldy,
                 const float* y_bias, void* out, float* state, long long slot_stride, const int* seq_slot,
                 const int* seq_q_start, const int* seq_q_len, int n_seqs, int max_q_len, int channels, cudaStream_t s) {
  if (n_seqs == 0 || channels == 0) return 0;
  if (bs < 1 || channels % bs || max_q_len < 1) return -2;
  // a warp a segment of at least 16 tokens, up to 32 warps
  int warps = max_q_len / 16;
  warps = warps < 1 ? 1 : warps > 32 ? 32 : warps;
  const dim3 grid(n_seqs, (channels + 31) / 32);
  if (dtype == 0)
    return launch_dependent(glru_scan_kernel<float>, grid, dim3(32 * warps), 0, s, (const float*)u, ldu, gates, n_tokens,
                            bs, r_bias, i_bias, lam, decay_scale, (const float*)ybranch, ldy, y_bias, (float*)out, state,
                            slot_stride, seq_slot, seq_q_start, seq_q_len, channels);
  return launch_dependent(glru_scan_kernel<bf16>, grid, dim3(32 * warps), 0, s, (const bf16*)u, ldu, gates, n_tokens, bs,
                          r_bias, i_bias, lam, decay_scale, (const bf16*)ybranch, ldy, y_bias, (bf16*)out, state,
                          slot_stride, seq_slot, seq_q_start, seq_q_len, channels);
}

}  // extern "C"
