// Grouped-query attention over the paged cache without rotation, whose positions enter through the
// scores and the mask instead:
//
//   score(i, j) = q_i . k_j * scale - r1_h * ln(1 + r2_h * (i - j))        a distance penalty per head
//   visible:      j <= i, and (chunk > 0) floor(i / chunk) == floor(j / chunk), and (window > 0) j > i - window;
//                 chunks are counted from position 0 of the sequence
//   softmax:      the denominator holds one more term exp(sink_h): a key that has no value
//   head output:  times gate[i, h], a number per token and head that arrives as sigmoid(g_h . x_i)
//
// Each of the four (penalty, chunk, sink, gate) is switched by its pointer or size, so a design may use
// any of them alone.  Keys have `dim` entries, values `vdim`.  Scores, the penalty with its logarithm,
// the running maximum and sum, the accumulator and the gate are float.
//
// The sink is the state the running softmax starts from: maximum = sink, sum = 1, accumulator = 0.
//
// Here: the kernel that files a step's keys and values and forms the gates (sink_prepare), and the plain
// attention kernel, one warp per (token, head), for the 32-bit path and for sizes the tensor-core kernel
// (attention_sink_tc.cu) does not take.
#include "common.cuh"

#define SINK_MAX_D 8  // dim, vdim <= 256

// proj: a row = [q (heads * dim) | k (kv_heads * dim) | v (kv_heads * vdim) | g (heads)]; without `write`
// the row has no k and v.  gate: float [tokens, heads] = sigmoid(g), or null when the row has no g.
template <typename T>
__global__ void sink_prepare_kernel(const T* __restrict__ proj, int proj_width, const int* __restrict__ tok_pos,
                                    const int* __restrict__ tok_slot, const int* __restrict__ block_table,
                                    int table_stride, T* __restrict__ k_store, T* __restrict__ v_store,
                                    float* __restrict__ gate, int heads, int kv_heads, int dim, int vdim, int write,
                                    int vec) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(proj);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(tok_slot);
  SB_BEHIND_WAIT(block_table);
  const int row = blockIdx.x;
  const T* pr = proj + (size_t)row * proj_width;
  const int q_width = heads * dim;
  int g_at = q_width;
  if (write) {
    const int pos = tok_pos[row];
    const int page = block_table[(size_t)tok_slot[row] * table_stride + pos / SB_PAGE_TOKENS];
    const int off = pos % SB_PAGE_TOKENS;
    const T* k = pr + q_width;
    const T* v = k + kv_heads * dim;
    constexpr int N = 16 / sizeof(T);       // entries of a 16-byte piece
    if (vec) {
      // rows, head sizes and bases in whole 16-byte pieces: a piece a thread
      for (int e = threadIdx.x; e < kv_heads * dim / N; e += blockDim.x) {
        const int h = e / (dim / N), d = (e - h * (dim / N)) * N;
        *reinterpret_cast<uint4*>(k_store + page_row(page, h, off, kv_heads, dim) + d) =
            *reinterpret_cast<const uint4*>(k + h * dim + d);
      }
      for (int e = threadIdx.x; e < kv_heads * vdim / N; e += blockDim.x) {
        const int h = e / (vdim / N), d = (e - h * (vdim / N)) * N;
        *reinterpret_cast<uint4*>(v_store + page_row(page, h, off, kv_heads, vdim) + d) =
            *reinterpret_cast<const uint4*>(v + h * vdim + d);
      }
    } else {
      for (int e = threadIdx.x; e < kv_heads * dim; e += blockDim.x) {
        const int h = e / dim, d = e - h * dim;
        k_store[page_row(page, h, off, kv_heads, dim) + d] = k[e];
      }
      for (int e = threadIdx.x; e < kv_heads * vdim; e += blockDim.x) {
        const int h = e / vdim, d = e - h * vdim;
        v_store[page_row(page, h, off, kv_heads, vdim) + d] = v[e];
      }
    }
    g_at += kv_heads * (dim + vdim);
  }
  if (gate)
    for (int h = threadIdx.x; h < heads; h += blockDim.x)
      gate[(size_t)row * heads + h] = 1.f / (1.f + expf(-to_f<T>(pr[g_at + h])));
}

// The same for a layer whose queries and keys are turned by their positions and whose values may be its keys:
// proj: a row = [q (heads * dim) | k (kv_heads * dim) | v (kv_heads * vdim), absent with v_from_k].  The first
// `rot` entries of every query and key head turn, entry 2i with entry 2i + 1, by the angle whose cos and sin
// stand at [position][i] of the float tables (rot / 2 columns; rot 0: nothing turns).  Queries are turned in
// place; keys go to the cache turned, values as they are; with v_from_k a key/value head's value is its key
// as projected, before the turn (vdim == dim).  A thread a pair of entries; the products are float.
template <typename T>
__global__ void sink_prepare_rot_kernel(T* __restrict__ proj, int proj_width, const int* __restrict__ tok_pos,
                                        const int* __restrict__ tok_slot, const int* __restrict__ block_table,
                                        int table_stride, T* __restrict__ k_store, T* __restrict__ v_store,
                                        const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot,
                                        int heads, int kv_heads, int dim, int vdim, int v_from_k, int write) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(proj);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(tok_slot);
  SB_BEHIND_WAIT(block_table);
  const int row = blockIdx.x;
  T* pr = proj + (size_t)row * proj_width;
  const int pos = tok_pos[row];
  const float* cr = cos_t + (size_t)pos * (rot / 2);
  const float* sr = sin_t + (size_t)pos * (rot / 2);
  const int half = (dim + 1) / 2;           // pairs a head (the last may be a single entry)
  for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
    const int h = e / half, i = e - h * half;
    if (2 * i + 1 >= dim || 2 * i >= rot) continue;
    T* at = pr + (size_t)h * dim + 2 * i;
    const float a = to_f<T>(at[0]), b = to_f<T>(at[1]), c = cr[i], s = sr[i];
    at[0] = from_f<T>(a * c - b * s);
    at[1] = from_f<T>(b * c + a * s);
  }
  if (!write) return;
  const int page = block_table[(size_t)tok_slot[row] * table_stride + pos / SB_PAGE_TOKENS];
  const int off = pos % SB_PAGE_TOKENS;
  const T* k = pr + (size_t)heads * dim;
  const T* v = k + (size_t)kv_heads * dim;
  for (int e = threadIdx.x; e < kv_heads * half; e += blockDim.x) {
    const int h = e / half, i = e - h * half;
    const bool two = 2 * i + 1 < dim;
    const float a = to_f<T>(k[(size_t)h * dim + 2 * i]), b = two ? to_f<T>(k[(size_t)h * dim + 2 * i + 1]) : 0.f;
    T* kd = k_store + page_row(page, h, off, kv_heads, dim) + 2 * i;
    if (two && 2 * i < rot) {
      const float c = cr[i], s = sr[i];
      kd[0] = from_f<T>(a * c - b * s);
      kd[1] = from_f<T>(b * c + a * s);
    } else {
      kd[0] = from_f<T>(a);
      if (two) kd[1] = from_f<T>(b);
    }
    if (v_from_k) {
      T* vd = v_store + page_row(page, h, off, kv_heads, vdim) + 2 * i;
      vd[0] = from_f<T>(a);
      if (two) vd[1] = from_f<T>(b);
    }
  }
  if (!v_from_k)
    for (int e = threadIdx.x; e < kv_heads * vdim; e += blockDim.x) {
      const int h = e / vdim, d = e - h * vdim;
      v_store[page_row(page, h, off, kv_heads, vdim) + d] = v[e];
    }
}

template <typename T>
__global__ void sink_attention_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out,
                                      const T* __restrict__ k_store, const T* __restrict__ v_store,
                                      const int* __restrict__ block_table, int table_stride,
                                      const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                                      const float* __restrict__ r1, const float* __restrict__ r2,
                                      const float* __restrict__ sink, const float* __restrict__ gate, int n_tokens,
                                      int heads, int kv_heads, int dim, int vdim, float scale, int chunk, int window) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(q);
  SB_BEHIND_WAIT(k_store);
  SB_BEHIND_WAIT(v_store);
  SB_BEHIND_WAIT(gate);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(tok_slot);
  SB_BEHIND_WAIT(block_table);
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)n_tokens * heads) return;
  const int token = (int)(warp / heads);
  const int h = (int)(warp - (long long)token * heads);
  const int kvh = h / (heads / kv_heads);
  const int pos = tok_pos[token];
  const int* pages = block_table + (size_t)tok_slot[token] * table_stride;
  const T* qr = q + (size_t)token * q_stride + (size_t)h * dim;

  float qv[SINK_MAX_D], acc[SINK_MAX_D];
#pragma unroll
  for (int i = 0; i < SINK_MAX_D; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < dim ? to_f<T>(qr[d]) : 0.f;
    acc[i] = 0.f;
  }
  const float pen1 = r1 ? r1[h] : 0.f, pen2 = r1 ? r2[h] : 0.f;
  float m = sink ? sink[h] : -INFINITY, l = sink ? 1.f : 0.f;
  int first = 0;
  if (chunk > 0) first = pos / chunk * chunk;
  if (window > 0 && pos - window + 1 > first) first = pos - window + 1;

  for (int j0 = first; j0 <= pos; j0 += 4) {
    float s[4];
    const T* vrow[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u;
      s[u] = 0.f;
      vrow[u] = nullptr;
      if (j <= pos) {
        const int page = pages[j / SB_PAGE_TOKENS];
        const T* kr = k_store + page_row(page, kvh, j % SB_PAGE_TOKENS, kv_heads, dim);
        vrow[u] = v_store + page_row(page, kvh, j % SB_PAGE_TOKENS, kv_heads, vdim);
#pragma unroll
        for (int i = 0; i < SINK_MAX_D; ++i) {
          const int d = lane + 32 * i;
          if (d < dim) s[u] += qv[i] * to_f<T>(kr[d]);
        }
      }
    }
    float m_new = m;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      s[u] = warp_sum(s[u]) * scale;
      if (r1) s[u] -= pen1 * log1pf(pen2 * (float)(pos - (j0 + u)));
      if (j0 + u <= pos) m_new = fmaxf(m_new, s[u]);
    }
    const float alpha = expf(m - m_new);
    l *= alpha;
#pragma unroll
    for (int i = 0; i < SINK_MAX_D; ++i) acc[i] *= alpha;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (j0 + u <= pos) {
        const float p = expf(s[u] - m_new);
        l += p;
#pragma unroll
        for (int i = 0; i < SINK_MAX_D; ++i) {
          const int d = lane + 32 * i;
          if (d < vdim) acc[i] += p * to_f<T>(vrow[u][d]);
        }
      }
    }
    m = m_new;
  }
  T* orow = out + ((size_t)token * heads + h) * vdim;
  const float inv = (gate ? gate[(size_t)token * heads + h] : 1.f) / l;
#pragma unroll
  for (int i = 0; i < SINK_MAX_D; ++i) {
    const int d = lane + 32 * i;
    if (d < vdim) orow[d] = from_f<T>(acc[i] * inv);
  }
}

extern "C" {

int sb_sink_max_dim() { return 32 * SINK_MAX_D; }

// proj: [n_tokens, proj_width]; k_store [pages, kv_heads, 64, dim], v_store [pages, kv_heads, 64, vdim]
// (ignored when write == 0); gate: float [n_tokens, heads] or null.
int sb_sink_prepare(int dtype, const void* proj, int proj_width, const int* tok_pos, const int* tok_slot,
                    const int* block_table, int table_stride, void* k_store, void* v_store, float* gate, int n_tokens,
                    int heads, int kv_heads, int dim, int vdim, int write, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if (proj_width < heads * dim + (write ? kv_heads * (dim + vdim) : 0) + (gate ? heads : 0)) return -2;
  const int n = dtype == 0 ? 4 : 8;
  const int vec = write && proj_width % n == 0 && dim % n == 0 && vdim % n == 0 &&
                  (((uintptr_t)proj | (uintptr_t)k_store | (uintptr_t)v_store) & 15) == 0;
  const int threads = write && vec && kv_heads * (dim + vdim) / n > 128 ? 256 : 128;
  if (dtype == 0)
    return launch_dependent(sink_prepare_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)proj, proj_width,
                            tok_pos, tok_slot, block_table, table_stride, (float*)k_store, (float*)v_store, gate, heads,
                            kv_heads, dim, vdim, write, vec);
  return launch_dependent(sink_prepare_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, (const bf16*)proj, proj_width,
                          tok_pos, tok_slot, block_table, table_stride, (bf16*)k_store, (bf16*)v_store, gate, heads,
                          kv_heads, dim, vdim, write, vec);
}

// proj: [n_tokens, proj_width], its queries turned in place; cos_t, sin_t: float [positions, rot / 2] (unused with
// rot 0); v_from_k: the row has no values and the keys as projected are filed as values (vdim == dim).
int sb_sink_prepare_rot(int dtype, void* proj, int proj_width, const int* tok_pos, const int* tok_slot,
                        const int* block_table, int table_stride, void* k_store, void* v_store, const float* cos_t,
                        const float* sin_t, int rot, int n_tokens, int heads, int kv_heads, int dim, int vdim,
                        int v_from_k, int write, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if (rot < 0 || rot % 2 || rot > dim || (v_from_k && vdim != dim)) return -2;
  if (proj_width < heads * dim + (write ? kv_heads * (dim + (v_from_k ? 0 : vdim)) : 0)) return -2;
  const int threads = heads * dim > 1024 ? 256 : 128;
  if (dtype == 0)
    return launch_dependent(sink_prepare_rot_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (float*)proj, proj_width,
                            tok_pos, tok_slot, block_table, table_stride, (float*)k_store, (float*)v_store, cos_t, sin_t,
                            rot, heads, kv_heads, dim, vdim, v_from_k, write);
  return launch_dependent(sink_prepare_rot_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, (bf16*)proj, proj_width,
                          tok_pos, tok_slot, block_table, table_stride, (bf16*)k_store, (bf16*)v_store, cos_t, sin_t, rot,
                          heads, kv_heads, dim, vdim, v_from_k, write);
}

// q: rows of q_stride entries whose first heads * dim are the queries; out: [n_tokens, heads * vdim].
// r1, r2: float [heads] or both null; sink: float [heads] or null; gate: float [n_tokens, heads] or null.
// chunk, window <= 0: none.
int sb_sink_attention(int dtype, const void* q, int q_stride, void* out, const void* k_store, const void* v_store,
                      const int* block_table, int table_stride, const int* tok_slot, const int* tok_pos,
                      const float* r1, const float* r2, const float* sink, const float* gate, int n_tokens, int heads,
                      int kv_heads, int dim, int vdim, float scale, int chunk, int window, cudaStream_t s) {
  if (dim > 32 * SINK_MAX_D || vdim > 32 * SINK_MAX_D || kv_heads <= 0 || heads % kv_heads) return -2;
  if ((r1 == nullptr) != (r2 == nullptr)) return -2;
  const long long warps = (long long)n_tokens * heads;
  if (warps == 0) return 0;
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  if (dtype == 0)
    return launch_dependent(sink_attention_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, s, (const float*)q,
                            q_stride, (float*)out, (const float*)k_store, (const float*)v_store, block_table,
                            table_stride, tok_slot, tok_pos, r1, r2, sink, gate, n_tokens, heads, kv_heads, dim, vdim,
                            scale, chunk, window);
  return launch_dependent(sink_attention_kernel<bf16>, dim3((unsigned)blocks), dim3(threads), 0, s, (const bf16*)q,
                          q_stride, (bf16*)out, (const bf16*)k_store, (const bf16*)v_store, block_table, table_stride,
                          tok_slot, tok_pos, r1, r2, sink, gate, n_tokens, heads, kv_heads, dim, vdim, scale, chunk,
                          window);
}

}  // extern "C"
