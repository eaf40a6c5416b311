// Linear recurrences with a matrix state S [N x V] per head, over the packed tokens of a step and the
// per-sequence state in the cache's slots, in two forms that share one kernel:
//
//   state-space (mode 0)   dt = softplus(a_raw + dt_bias), g = exp(-exp(A_log) dt)
//                          S <- g S + k (dt v)^T,   o = S^T q + D v              (k = B, q = C, v = x)
//   gated delta (mode 1)   g = exp(-exp(A_log) softplus(a_raw + dt_bias)), beta = sigmoid(b_raw)
//                          q <- q / sqrt(sum q^2 + 1e-6) * N^-1/2,  k <- k / sqrt(sum k^2 + 1e-6)
//                          S <- g S,  u = beta (v - S^T k),  S <- S + k u^T,  o = S^T q
//
// q and k have `G` heads; head h reads head h / (H / G).  S is float in the slot ([H][N][V]), from zero for a
// new sequence.  Everything but the loads of q, k, v, a_raw, b_raw (working type T) is float; o is stored float.
//
// A block owns 32 columns of one head's S for one sequence: 256 threads = 32 columns x 8 lanes; lane p of a
// column keeps rows p, p + 8, ... (KPT of them) in registers, and the eight lanes of a column sum S^T k and
// S^T q by shuffles.  (States of more than 64 rows: 16 columns x 16 lanes.)  Both are taken from the state as the token finds it: with u the token's write,
// (g S + k u^T)^T q = g S^T q + u (k . q), so one round of shuffles a token serves both and the decay is folded
// into the write.  Tokens arrive in chunks of 16 through two shared-memory buffers (q, k as floats, padded with
// zeros to 8 * KPT rows; k . q and the unit norms are taken there, a warp a token); the next chunk's global
// loads are issued before the current chunk is walked and filed after it; outputs leave through shared memory.
//
// Also here: the RMS norm in equal parts of a row with a gate (group_norm_gate), and the mean of two rows each
// RMS-normed with a gain of its own (norm_pair_mean).
#include "common.cuh"

#define SCAN_CT 16
#define SCAN_MAX_N 256

__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// The sum over the P neighbouring lanes that share a column (P = 8 or 16).
template <int P> __device__ __forceinline__ float sum_lanes(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  if (P == 16) v += __shfl_xor_sync(0xffffffffu, v, 8);
  return v;
}

// Shared memory of one buffer of SCAN_CT tokens: q and k as floats (NP entries a token), the block's 32 value
// columns, and per token the decay, the factor (dt, or beta) and k . q.
template <int NP, int COLS> struct ScanBuffer {
  float q[SCAN_CT][NP], k[SCAN_CT][NP], v[SCAN_CT][COLS], dec[SCAN_CT], fac[SCAN_CT], kq[SCAN_CT];   // dec: 1 - decay
};

template <typename T, int MODE, int KPT, int P>
__global__ void __launch_bounds__(256)
state_scan_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k, int ldk, const T* __restrict__ v, int ldv,
                  const T* __restrict__ a_raw, int lda, const T* __restrict__ b_raw, int ldb,
                  const float* __restrict__ A_log, const float* __restrict__ dt_bias, const float* __restrict__ D,
                  float* __restrict__ state, long long slot_stride, float* __restrict__ out,
                  const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                  const int* __restrict__ seq_q_len, int H, int G, int N, int V) {
  constexpr int NP = P * KPT, SCAN_COLS = 256 / P;
  constexpr int QK_PER = (SCAN_CT * NP + 255) / 256, V_PER = SCAN_CT * SCAN_COLS / 256;
  typedef ScanBuffer<NP, SCAN_COLS> Buffer;
  extern __shared__ __align__(16) unsigned char scan_smem[];
  Buffer* bufs = reinterpret_cast<Buffer*>(scan_smem);
  float (*os)[SCAN_COLS] = reinterpret_cast<float (*)[SCAN_COLS]>(scan_smem + 2 * sizeof(Buffer));
  // (launch_dependents comes at this kernel's end, not its start: a long prompt keeps its blocks for a while)
  pdl_wait();
  SB_BEHIND_WAIT(q);
  SB_BEHIND_WAIT(k);
  SB_BEHIND_WAIT(v);
  SB_BEHIND_WAIT(a_raw);
  SB_BEHIND_WAIT(b_raw);
  SB_BEHIND_WAIT(state);
  SB_BEHIND_WAIT(seq_slot);
  SB_BEHIND_WAIT(seq_q_start);
  SB_BEHIND_WAIT(seq_q_len);
  const int seq = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * SCAN_COLS;
  const int tid = threadIdx.x, p = tid & (P - 1), jj = tid / P, lane = tid & 31, warp = tid >> 5;
  const int g = h / (H / G);
  const int q_start = seq_q_start[seq], q_len = seq_q_len[seq];
  float* sp = state + (size_t)seq_slot[seq] * slot_stride + (size_t)h * N * V;
  const int j = col0 + jj;
  const bool col = j < V;
  float S[KPT];
#pragma unroll
  for (int r = 0; r < KPT; ++r) {
    const int i = p + P * r;
    S[r] = (col && i < N) ? sp[(size_t)i * V + j] : 0.f;
  }
  const float rate = expf(A_log[h]), bias = dt_bias[h], skip = (MODE == 0 && D) ? D[h] : 0.f;
  const float q_mult = MODE == 1 ? rsqrtf((float)N) : 1.f;

  // a chunk's loads, held in registers while the chunk before is walked
  T rq[QK_PER], rk[QK_PER], rv[V_PER];
  float ra = 0.f, rb = 0.f;
  auto fetch = [&](int t0) {
    const int ct = min(SCAN_CT, q_len - t0);
#pragma unroll
    for (int n = 0; n < QK_PER; ++n) {
      const int e = tid + 256 * n, tt = e / NP, i = e - tt * NP;
      const bool have = tt < ct && i < N;
      const size_t row = (size_t)(q_start + t0 + (have ? tt : 0));
      rq[n] = have ? q[row * ldq + (size_t)g * N + i] : from_f<T>(0.f);
      rk[n] = have ? k[row * ldk + (size_t)g * N + i] : from_f<T>(0.f);
    }
#pragma unroll
    for (int n = 0; n < V_PER; ++n) {
      const int e = tid + 256 * n, tt = e / SCAN_COLS, c = e - tt * SCAN_COLS;
      const bool have = tt < ct && col0 + c < V;
      rv[n] = have ? v[(size_t)(q_start + t0 + tt) * ldv + (size_t)h * V + col0 + c] : from_f<T>(0.f);
    }
    if (tid < ct) {
      const size_t row = (size_t)(q_start + t0 + tid);
      ra = to_f<T>(a_raw[row * lda + h]);
      if (MODE == 1) rb = to_f<T>(b_raw[row * ldb + h]);
    }
  };
  // the registers into a buffer, then (behind a barrier) per token k . q and, for the delta rule, the unit vectors
  auto file = [&](Buffer& b, int t0) {
    const int ct = min(SCAN_CT, q_len - t0);
#pragma unroll
    for (int n = 0; n < QK_PER; ++n) {
      const int e = tid + 256 * n;
      if (e < SCAN_CT * NP) {
        (&b.q[0][0])[e] = to_f<T>(rq[n]);
        (&b.k[0][0])[e] = to_f<T>(rk[n]);
      }
    }
#pragma unroll
    for (int n = 0; n < V_PER; ++n) (&b.v[0][0])[tid + 256 * n] = to_f<T>(rv[n]);
    if (tid < ct) {
      const float dt = softplus_f(ra + bias);
      b.dec[tid] = -expm1f(-rate * dt);        // the decay's complement 1 - g: see the walk
      b.fac[tid] = MODE == 0 ? dt : 1.f / (1.f + expf(-rb));
    }
    __syncthreads();
    for (int tt = warp; tt < ct; tt += 8) {
      float sq = 0.f, sk = 0.f, dot = 0.f;
      for (int i = lane; i < NP; i += 32) {
        const float a = b.q[tt][i], c = b.k[tt][i];
        sq += a * a;
        sk += c * c;
        dot += a * c;
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      dot = warp_sum(dot);
      if (MODE == 1) {
        const float mq = q_mult / sqrtf(sq + 1e-6f), mk = 1.f / sqrtf(sk + 1e-6f);
        for (int i = lane; i < NP; i += 32) {
          b.q[tt][i] *= mq;
          b.k[tt][i] *= mk;
        }
        dot *= mq * mk;
      }
      if (lane == 0) b.kq[tt] = dot;
    }
    __syncthreads();
  };

  fetch(0);
  file(bufs[0], 0);
  int which = 0;
  for (int t0 = 0; t0 < q_len; t0 += SCAN_CT, which ^= 1) {
    const int ct = min(SCAN_CT, q_len - t0);
    const bool more = t0 + SCAN_CT < q_len;
    if (more) fetch(t0 + SCAN_CT);
    const Buffer& b = bufs[which];
    for (int tt = 0; tt < ct; ++tt) {
      // both read-outs come from the state as the token finds it: with u the token's write,
      // (g S + k u^T)^T q = g S^T q + u (k . q), so one round of shuffles a token serves both
      // (the decay g arrives as d = 1 - g and is applied as S - d * S: a g close to one, rounded to a float,
      // would lose up to 2^-24 / (1 - g) of the decay's rate)
      const float dd = b.dec[tt], x = b.v[tt][jj];
      float kk[KPT], r1a = 0.f, r1b = 0.f, r2a = 0.f, r2b = 0.f;
#pragma unroll
      for (int r = 0; r < KPT; ++r) {
        kk[r] = b.k[tt][p + P * r];
        const float qq = b.q[tt][p + P * r];
        if (r & 1) {
          if (MODE == 1) r1b += S[r] * kk[r];
          r2b += S[r] * qq;
        } else {
          if (MODE == 1) r1a += S[r] * kk[r];
          r2a += S[r] * qq;
        }
      }
      float r1 = r1a + r1b, r2 = r2a + r2b;
      r2 = sum_lanes<P>(r2);
      float u;
      if (MODE == 1) {
        r1 = sum_lanes<P>(r1);
        u = b.fac[tt] * (x - fmaf(-dd, r1, r1));
      } else {
        u = b.fac[tt] * x;
      }
#pragma unroll
      for (int r = 0; r < KPT; ++r) S[r] = fmaf(kk[r], u, fmaf(-dd, S[r], S[r]));
      if (p == 0) os[tt][jj] = fmaf(-dd, r2, r2) + u * b.kq[tt] + skip * x;
    }
    __syncthreads();
    for (int e = tid; e < ct * SCAN_COLS; e += 256) {
      const int tt = e / SCAN_COLS, c = e - tt * SCAN_COLS;
      if (col0 + c < V) out[(size_t)(q_start + t0 + tt) * H * V + (size_t)h * V + col0 + c] = os[tt][c];
    }
    if (more) file(bufs[which ^ 1], t0 + SCAN_CT);      // (its barriers also keep os until it is stored)
    else __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < KPT; ++r) {
    const int i = p + P * r;
    if (col && i < N) sp[(size_t)i * V + j] = S[r];
  }
}

// ------------------------------------------------------------------------------------------ norm in parts, gated
// A warp a (token, part).  order 0: y = rms(o * silu(z)) * w (the gate in front of the norm); order 1:
// y = rms(o) * w * silu(z).  w has `wlen` entries and is read at (column mod wlen): a gain of the whole row,
// or one of a part's size that every part shares.
// WIDE: a block a (token, part) instead, for parts of many entries.
template <typename T, bool WIDE>
__global__ void group_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ z, int ldz,
                                       const float* __restrict__ w, int wlen, T* __restrict__ y, int n_tokens,
                                       int parts, int psize, float eps, int order) {
  __shared__ float scratch[33];
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(o);
  SB_BEHIND_WAIT(z);
  const long long item = WIDE ? (long long)blockIdx.x : ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = WIDE ? threadIdx.x : threadIdx.x & 31;
  const int step = WIDE ? blockDim.x : 32;
  if (item >= (long long)n_tokens * parts) return;
  const int token = (int)(item / parts), part = (int)(item - (long long)token * parts);
  const float* orow = o + (size_t)token * parts * psize + (size_t)part * psize;
  const T* zrow = z + (size_t)token * ldz + (size_t)part * psize;
  float sq = 0.f;
  for (int c = lane; c < psize; c += step) {
    float val = orow[c];
    if (order == 0) {
      const float gz = to_f<T>(zrow[c]);
      val *= gz / (1.f + expf(-gz));
    }
    sq += val * val;
  }
  sq = WIDE ? block_sum(sq, scratch) : warp_sum(sq);
  const float inv = 1.f / sqrtf(sq / (float)psize + eps);
  T* yrow = y + (size_t)token * parts * psize + (size_t)part * psize;
  for (int c = lane; c < psize; c += step) {
    const float gz = to_f<T>(zrow[c]);
    const float silu = gz / (1.f + expf(-gz));
    const float gain = w[(part * psize + c) % wlen];
    yrow[c] = from_f<T>(order == 0 ? orow[c] * silu * inv * gain : orow[c] * inv * gain * silu);
  }
}

// out = (rms(a) * wa + rms(b) * wb) / 2, a block a row.
template <typename T>
__global__ void norm_pair_mean_kernel(const T* __restrict__ a, const T* __restrict__ b, const float* __restrict__ wa,
                                      const float* __restrict__ wb, T* __restrict__ out, int width, float eps) {
  __shared__ float scratch[33];
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(a);
  SB_BEHIND_WAIT(b);
  const T* ar = a + (size_t)blockIdx.x * width;
  const T* br = b + (size_t)blockIdx.x * width;
  float sa = 0.f, sb = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float x = to_f<T>(ar[c]), y = to_f<T>(br[c]);
    sa += x * x;
    sb += y * y;
  }
  sa = block_sum(sa, scratch);
  sb = block_sum(sb, scratch);
  const float ia = 1.f / sqrtf(sa / (float)width + eps), ib = 1.f / sqrtf(sb / (float)width + eps);
  T* orow = out + (size_t)blockIdx.x * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    orow[c] = from_f<T>(0.5f * (to_f<T>(ar[c]) * ia * wa[c] + to_f<T>(br[c]) * ib * wb[c]));
}

template <typename T, int MODE>
static int scan_launch(int kpt, int lanes, int n_seqs, cudaStream_t s, const void* q, int ldq, const void* k, int ldk,
                       const void* v, int ldv, const void* a_raw, int lda, const void* b_raw, int ldb, const float* A_log,
                       const float* dt_bias, const float* D, float* state, long long slot_stride, float* out,
                       const int* seq_slot, const int* seq_q_start, const int* seq_q_len, int H, int G, int N, int V) {
#define SCAN_GO(KPT, P)                                                                                                \
  {                                                                                                                    \
    const size_t smem = 2 * sizeof(ScanBuffer<P * KPT, 256 / P>) + SCAN_CT * (256 / P) * sizeof(float);                 \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(state_scan_kernel<T, MODE, KPT, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    const dim3 grid(n_seqs, H, (V + 256 / P - 1) / (256 / P));                                                         \
    return launch_dependent(state_scan_kernel<T, MODE, KPT, P>, grid, dim3(256), smem, s, (const T*)q, ldq,             \
                            (const T*)k, ldk, (const T*)v, ldv, (const T*)a_raw, lda, (const T*)b_raw, ldb, A_log,      \
                            dt_bias, D, state, slot_stride, out, seq_slot, seq_q_start, seq_q_len, H, G, N, V);         \
  }
  if (lanes == 16) {
    if (kpt == 8) SCAN_GO(8, 16)
    SCAN_GO(16, 16)
  }
  switch (kpt) {
    case 1: SCAN_GO(1, 8)
    case 2: SCAN_GO(2, 8)
    case 4: SCAN_GO(4, 8)
    case 8: SCAN_GO(8, 8)
    default: SCAN_GO(16, 8)
  }
#undef SCAN_GO
}

extern "C" {

int sb_scan_max_state() { return SCAN_MAX_N; }

// mode 0: state-space; 1: gated delta.  q, k: [n_tokens, ld] with G heads of N entries from the pointer on;
// v: H heads of V; a_raw (and b_raw in mode 1): H entries; A_log, dt_bias (and D in mode 0, or null): float
// [H]; state: float, a slot's [H][N][V] starts at the pointer; out: float [n_tokens, H * V].
int sb_state_scan(int dtype, int mode, const void* q, int ldq, const void* k, int ldk, const void* v, int ldv,
                  const void* a_raw, int lda, const void* b_raw, int ldb, const float* A_log, const float* dt_bias,
                  const float* D, float* state, long long slot_stride, float* out, const int* seq_slot,
                  const int* seq_q_start, const int* seq_q_len, int n_seqs, int H, int G, int N, int V, cudaStream_t s) {
  if (n_seqs == 0) return 0;
  if (N < 1 || N > SCAN_MAX_N || V < 1 || H < 1 || G < 1 || H % G || (mode != 0 && mode != 1)) return -2;
  if (mode == 1 && !b_raw) return -2;
  // 8 lanes a column and 32 columns a block; for states of more than 64 rows in a step whose blocks would not
  // fill the SMs twice (a prompt of one or two sequences), 16 lanes and 16 columns: half the rows a thread, twice
  // the blocks, a shorter chain of sums a token
  const long long blocks8 = (long long)n_seqs * H * ((V + 31) / 32);
  const int lanes = N > 128 || (N > 64 && blocks8 < 2 * 148) ? 16 : 8;
  int kpt = lanes == 16 ? 8 : 1;
  while (lanes * kpt < N) kpt *= 2;
#define SCAN_ARGS kpt, lanes, n_seqs, s, q, ldq, k, ldk, v, ldv, a_raw, lda, b_raw, ldb, A_log, dt_bias, D, state, slot_stride, out, \
                  seq_slot, seq_q_start, seq_q_len, H, G, N, V
  if (dtype == 0) return mode == 0 ? scan_launch<float, 0>(SCAN_ARGS) : scan_launch<float, 1>(SCAN_ARGS);
  return mode == 0 ? scan_launch<bf16, 0>(SCAN_ARGS) : scan_launch<bf16, 1>(SCAN_ARGS);
#undef SCAN_ARGS
}

// o: float [n_tokens, parts * psize]; z: [n_tokens, ldz] (working type, the gate's entries from the pointer on);
// w: float [wlen]; y: [n_tokens, parts * psize].  order 0: gate, then norm; 1: norm, then gate.
int sb_group_norm_gate(int dtype, const float* o, const void* z, int ldz, const float* w, int wlen, void* y, int n_tokens,
                       int parts, int psize, float eps, int order, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if (parts < 1 || psize < 1 || wlen < 1 || (order != 0 && order != 1)) return -2;
  const long long warps = (long long)n_tokens * parts;
  if (psize > 256) {
    const dim3 grid((unsigned)warps), block(psize >= 1024 ? 256 : 128);
    if (dtype == 0)
      return launch_dependent(group_norm_gate_kernel<float, true>, grid, block, 0, s, o, (const float*)z, ldz, w, wlen,
                              (float*)y, n_tokens, parts, psize, eps, order);
    return launch_dependent(group_norm_gate_kernel<bf16, true>, grid, block, 0, s, o, (const bf16*)z, ldz, w, wlen,
                            (bf16*)y, n_tokens, parts, psize, eps, order);
  }
  const dim3 grid((unsigned)((warps + 7) / 8));
  if (dtype == 0)
    return launch_dependent(group_norm_gate_kernel<float, false>, grid, dim3(256), 0, s, o, (const float*)z, ldz, w, wlen,
                            (float*)y, n_tokens, parts, psize, eps, order);
  return launch_dependent(group_norm_gate_kernel<bf16, false>, grid, dim3(256), 0, s, o, (const bf16*)z, ldz, w, wlen,
                          (bf16*)y, n_tokens, parts, psize, eps, order);
}

int sb_norm_pair_mean(int dtype, const void* a, const void* b, const float* wa, const float* wb, void* out, int n_tokens,
                      int width, float eps, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  const int threads = width >= 2048 ? 512 : width >= 512 ? 256 : 128;
  if (dtype == 0)
    return launch_dependent(norm_pair_mean_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)a,
                            (const float*)b, wa, wb, (float*)out, width, eps);
  return launch_dependent(norm_pair_mean_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, (const bf16*)a, (const bf16*)b,
                          wa, wb, (bf16*)out, width, eps);
}

}  // extern "C"
