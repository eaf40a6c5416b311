// A routed mixture of small gated feed-forward experts, for any number of tokens, without a word
// from the host between its kernels (so that it can sit inside a captured step).
//
//   route    z = W_r h + b in float; the `top` largest (the lower index first among equals); their
//            weights are the softmax over those `top` logits alone (scoring 0), or their sigmoids divided
//            by the sum of those sigmoids (+ 1e-20) and multiplied by a constant (scoring 1).
//   align    the (token, choice) pairs grouped by expert: every expert's pairs fill whole tiles of
//            rows (32, or 64 for the tensor-core tiles; padded with -1), `tile_expert` names each tile's expert, `n_tiles` counts them.
//   up       per tile: g = min(gate(h), limit), u = clamp(up(h), -limit, limit),
//            a = g * sigmoid(1.702 g) * (u + 1), for the tile's rows gathered from h (expert kind 1);
//            or, for experts without a gate, a = relu(up(h))^2 (expert kind 2); with limit 0 the gated kind
//            has no clamps and the plain gate: a = silu(gate(h)) * up(h).
//   down     per tile: the expert's down projection of a, filed at the pair's own place.
//   combine  out[t] = sum_c weight[t][c] * down[t][c], summed in float in the order of the choices.
//
// A second router (route_all) scores by the softmax over ALL its outputs, chooses by score + correction among the
// experts of the best groups, and may have more outputs than there are experts: a choice from `experts` on is
// an identity expert, which has no weights.  align leaves such pairs out of the tiles and combine adds the
// token's own row in their place.  combine also adds a shared expert's output times a gate per token.
//
// Products accumulate in float; gate and up are rounded to the working type before the activation, as
// the projections of the dense feed-forward are.  A token's result depends on nothing but its own row
// and the experts' weights: not on which tile it landed in, nor on who else is in the step.
#include <mma.h>

#include "common.cuh"

#define MOE_BM 32
#define MOE_BN 64
#define MOE_BK 32
#define MOE_MAX_EXPERTS 1024
#define MOE_MAX_TOP 16

// The gated expert's activation from its (rounded) gate and up products.  limit > 0: the clamped gate,
// min(g, limit) * sigmoid(1.702 min(g, limit)) * (clamp(u, -limit, limit) + 1); limit == 0: no clamps and the
// plain gate silu(g) * u.
__device__ __forceinline__ float moe_gate(float g, float u, float limit) {
  if (limit > 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
  }
  return g / (1.f + expf(-g)) * u;
}

template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, const float* __restrict__ w, const float* __restrict__ b,
                                 int* __restrict__ ids, float* __restrict__ weights, int width, int experts, int top,
                                 int scoring, float weight_scale) {
  extern __shared__ float z[];
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(h);
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const T* hr = h + (size_t)row * width;
  // (16-byte pieces of the router's rows when the rows allow it: a lane's loads are then all in flight together)
  const bool wide = width % 4 == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)hr % 8) == 0;
  for (int e = warp; e < experts; e += warps) {
    const float* wr = w + (size_t)e * width;
    float a = 0.f;
    if (wide && sizeof(T) == 2) {
      const float4* w4 = reinterpret_cast<const float4*>(wr);
      const uint2* h4 = reinterpret_cast<const uint2*>(hr);
#pragma unroll 4
      for (int c = lane; c < width / 4; c += 32) {
        const float4 wv = w4[c];
        const uint2 hv = h4[c];
        a += __uint_as_float(hv.x << 16) * wv.x + __uint_as_float(hv.x & 0xffff0000u) * wv.y +
             __uint_as_float(hv.y << 16) * wv.z + __uint_as_float(hv.y & 0xffff0000u) * wv.w;
      }
    } else {
      for (int c = lane; c < width; c += 32) a += to_f<T>(hr[c]) * wr[c];
    }
    a = warp_sum(a);
    if (lane == 0) z[e] = a + (b ? b[e] : 0.f);
  }
  __syncthreads();
  if (warp == 0) {
    float best[MOE_MAX_TOP];
    float top_max = 0.f;
    for (int c = 0; c < top; ++c) {
      // the largest logit left, the lowest index among equals
      float v = -INFINITY;
      int at = 0x7fffffff;
      for (int e = lane; e < experts; e += 32)
        if (z[e] > v) { v = z[e]; at = e; }
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ov > v || (ov == v && oa < at)) { v = ov; at = oa; }
      }
      if (at >= experts) at = 0;          // no finite logit left: keep the indices inside the table
      if (c == 0) top_max = v;
      best[c] = v;
      if (lane == 0) {
        ids[(size_t)row * top + c] = at;
        z[at] = -INFINITY;
      }
      __syncwarp();
    }
    if (lane == 0) {
      float sum = 0.f;
      for (int c = 0; c < top; ++c) {
        best[c] = scoring == 1 ? 1.f / (1.f + expf(-best[c])) : expf(best[c] - top_max);
        sum += best[c];
      }
      if (scoring == 1) {
        for (int c = 0; c < top; ++c) weights[(size_t)row * top + c] = best[c] / (sum + 1e-20f) * weight_scale;
      } else {
        for (int c = 0; c < top; ++c) weights[(size_t)row * top + c] = best[c] / sum;
      }
    }
  }
}

// The router of the softmax over all outputs (see sb_moe_route_all).  z holds outputs + 1 logits (the last one
// the shared expert's gate, when asked for), then the scores, the choice numbers and the groups' maxima.
template <typename T>
__global__ void moe_route_all_kernel(const T* __restrict__ h, const float* __restrict__ w,
                                     const float* __restrict__ correction, int* __restrict__ ids,
                                     float* __restrict__ weights, float* __restrict__ gate_out, int width, int outputs,
                                     int top, int groups, int keep, float weight_scale) {
  extern __shared__ float z[];
  float* score = z + outputs + 1;
  float* choice = score + outputs;
  float* best_of = choice + outputs;
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(h);
  const int row = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const T* hr = h + (size_t)row * width;
  const int rows = outputs + (gate_out ? 1 : 0);
  const bool wide = width % 4 == 0 && ((uintptr_t)w % 16) == 0 && ((uintptr_t)hr % 8) == 0;
  for (int e = warp; e < rows; e += warps) {
    const float* wr = w + (size_t)e * width;
    float a = 0.f;
    if (wide && sizeof(T) == 2) {
      const float4* w4 = reinterpret_cast<const float4*>(wr);
      const uint2* h4 = reinterpret_cast<const uint2*>(hr);
#pragma unroll 4
      for (int c = lane; c < width / 4; c += 32) {
        const float4 wv = w4[c];
        const uint2 hv = h4[c];
        a += __uint_as_float(hv.x << 16) * wv.x + __uint_as_float(hv.x & 0xffff0000u) * wv.y +
             __uint_as_float(hv.y << 16) * wv.z + __uint_as_float(hv.y & 0xffff0000u) * wv.w;
      }
    } else {
      for (int c = lane; c < width; c += 32) a += to_f<T>(hr[c]) * wr[c];
    }
    a = warp_sum(a);
    if (lane == 0) z[e] = a;
  }
  __syncthreads();
  if (warp != 0) return;
  if (gate_out && lane == 0) gate_out[row] = 1.f / (1.f + expf(-z[outputs]));
  float top_z = -INFINITY;
  for (int e = lane; e < outputs; e += 32) top_z = fmaxf(top_z, z[e]);
  top_z = warp_max(top_z);
  float sum = 0.f;
  for (int e = lane; e < outputs; e += 32) {
    const float v = expf(z[e] - top_z);
    score[e] = v;
    sum += v;
  }
  sum = warp_sum(sum);
  for (int e = lane; e < outputs; e += 32) {
    score[e] /= sum;
    choice[e] = score[e] + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (groups > 1) {
    const int per = outputs / groups;
    for (int g = lane; g < groups; g += 32) {
      float v = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) v = fmaxf(v, choice[e]);
      best_of[g] = v;
    }
    __syncwarp();
    // the `keep` best groups are marked with +inf, then every other group's outputs leave the choice
    for (int c = 0; c < keep; ++c) {
      float v = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (best_of[g] != INFINITY && (best_of[g] > v || at == 0x7fffffff)) { v = best_of[g]; at = g; }
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa != 0x7fffffff && (at == 0x7fffffff || ov > v || (ov == v && oa < at))) { v = ov; at = oa; }
      }
      if (lane == 0 && at < groups) best_of[at] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < outputs; e += 32)
      if (best_of[e / per] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  float picked[MOE_MAX_TOP];
  for (int c = 0; c < top; ++c) {
    float v = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < outputs; e += 32)
      if (choice[e] > v) { v = choice[e]; at = e; }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ov > v || (ov == v && oa < at)) { v = ov; at = oa; }
    }
    if (at >= outputs) at = 0;          // nothing left to choose from: keep the indices inside the table
    picked[c] = score[at];
    if (lane == 0) {
      ids[(size_t)row * top + c] = at;
      choice[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane == 0) {
    float total = 0.f;
    for (int c = 0; c < top; ++c) total += picked[c];
    for (int c = 0; c < top; ++c) weights[(size_t)row * top + c] = picked[c] / (total + 1e-20f) * weight_scale;
  }
}

// One block.  ids: [n_pairs]; sorted: [capacity] receives pair numbers or -1; tile_expert: [max_tiles].
__global__ void moe_align_kernel(const int* __restrict__ ids, int n_pairs, int experts, int* __restrict__ sorted,
                                 int capacity, int* __restrict__ tile_expert, int* __restrict__ n_tiles, int bm) {
  __shared__ int count[MOE_MAX_EXPERTS], offset[MOE_MAX_EXPERTS], total;
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(ids);
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  // (an id from `experts` on names an identity expert: it has no tile)
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x)
    if (ids[i] < experts) atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0, tiles = 0;
    for (int e = 0; e < experts; ++e) {
      offset[e] = off;
      const int nt = (count[e] + bm - 1) / bm;
      for (int t = 0; t < nt; ++t) tile_expert[tiles++] = e;
      off += nt * bm;
      count[e] = 0;
    }
    n_tiles[0] = tiles;
    total = off;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < total && i < capacity; i += blockDim.x) sorted[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e < experts) sorted[offset[e] + atomicAdd(&count[e], 1)] = i;
  }
}

// A tile of MOE_BM rows times MOE_BN outputs in float on the CUDA cores: the 32-bit path, and the
// working-type path for widths the tensor-core kernel does not take.  MODE 1: rows gathered from h by
// pair / top, two weight blocks (gate, up) and the gated activation; MODE 2: rows gathered likewise, one
// weight block, squared relu; MODE 0: rows of `a`, one block, results filed by pair.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_tile_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, const int* __restrict__ sorted,
                const int* __restrict__ tile_expert, const int* __restrict__ n_tiles, int k_dim, int n_out, int top,
                float limit) {
  __shared__ float xs[MOE_BM][MOE_BK + 1];
  constexpr bool UP = MODE != 0;
  constexpr int NW = MODE == 1 ? 2 : 1;
  __shared__ float ws[NW][MOE_BN][MOE_BK + 1];
  __shared__ int src[MOE_BM];
  // (launch_dependents comes at this kernel's end, not its start: it runs in several waves of large blocks,
  // and a successor that starts early would only sit on the SMs its later waves need)
  pdl_wait();
  SB_BEHIND_WAIT(x);
  SB_BEHIND_WAIT(sorted);
  SB_BEHIND_WAIT(tile_expert);
  SB_BEHIND_WAIT(n_tiles);
  const int tile = blockIdx.x;
  if (tile >= n_tiles[0]) return;
  const int e = tile_expert[tile];
  const int n0 = blockIdx.y * MOE_BN;
  const int tid = threadIdx.x;
  if (tid < MOE_BM) src[tid] = sorted[tile * MOE_BM + tid];
  __syncthreads();
  const T* we = w + (size_t)e * NW * n_out * k_dim;
  const int ty = tid >> 4, tx = tid & 15;
  float acc[NW][2][4];
#pragma unroll
  for (int a = 0; a < NW; ++a)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[a][i][j] = 0.f;
  for (int k0 = 0; k0 < k_dim; k0 += MOE_BK) {
    for (int i = tid; i < MOE_BM * MOE_BK; i += 256) {
      const int m = i / MOE_BK, kk = i % MOE_BK;
      const int pair = src[m];
      float v = 0.f;
      if (pair >= 0 && k0 + kk < k_dim) {
        const size_t row = UP ? (size_t)(pair / top) : (size_t)tile * MOE_BM + m;
        v = to_f<T>(x[row * k_dim + k0 + kk]);
      }
      xs[m][kk] = v;
    }
    for (int i = tid; i < NW * MOE_BN * MOE_BK; i += 256) {
      const int a = i / (MOE_BN * MOE_BK), rem = i % (MOE_BN * MOE_BK);
      const int n = rem / MOE_BK, kk = rem % MOE_BK;
      float v = 0.f;
      if (n0 + n < n_out && k0 + kk < k_dim) v = to_f<T>(we[((size_t)a * n_out + n0 + n) * k_dim + k0 + kk]);
      ws[a][n][kk] = v;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < MOE_BK; ++kk) {
      const float x0 = xs[ty * 2][kk], x1 = xs[ty * 2 + 1][kk];
#pragma unroll
      for (int a = 0; a < NW; ++a)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float wv = ws[a][tx + 16 * j][kk];
          acc[a][0][j] += x0 * wv;
          acc[a][1][j] += x1 * wv;
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int m = ty * 2 + i;
    const int pair = src[m];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= n_out) continue;
      if (MODE == 1) {
        const float g = rnd<T>(acc[0][i][j]), u = rnd<T>(acc[NW - 1][i][j]);
        const float a = pair >= 0 ? moe_gate(g, u, limit) : 0.f;
        y[((size_t)tile * MOE_BM + m) * n_out + n] = from_f<T>(a);
      } else if (MODE == 2) {
        const float u = fmaxf(rnd<T>(acc[0][i][j]), 0.f);
        y[((size_t)tile * MOE_BM + m) * n_out + n] = from_f<T>(pair >= 0 ? u * u : 0.f);
      } else if (pair >= 0) {
        y[(size_t)pair * n_out + n] = from_f<T>(acc[0][i][j]);
      }
    }
  }
}

// The same on the tensor cores (bfloat16, k a multiple of 16): tiles of 64 rows times 64 outputs, eight
// warps (four groups of 16 rows times two halves of the outputs), wmma 16 x 16 x 16 with float
// accumulators.  Rows (gathered through `sorted`) and weights arrive in k-slices of 64 through a ring of
// three cp.async stages, so that the copies of the next two slices are in flight while one is multiplied.
#define MOE_TC_BM 64
#define MOE_TC_BK 64
__device__ __forceinline__ void moe_cp16(void* dst, const void* src, bool real) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = real ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(256)
moe_tile_tc_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                   const int* __restrict__ sorted, const int* __restrict__ tile_expert,
                   const int* __restrict__ n_tiles, int k_dim, int n_out, int top, float limit) {
  using namespace nvcuda;
  constexpr bool UP = MODE != 0;
  constexpr int BK = MOE_TC_BK, LD = BK + 8, NW = MODE == 1 ? 2 : 1, STAGES = 3, CLD = MOE_BN + 4;
  constexpr int PIECES = BK / 8, PASS_ROWS = 256 / PIECES, PASSES = MOE_TC_BM / PASS_ROWS;
  extern __shared__ __align__(128) unsigned char moe_smem[];
  bf16* xs = reinterpret_cast<bf16*>(moe_smem);                          // [STAGES][64][LD]
  bf16* ws = xs + STAGES * MOE_TC_BM * LD;                               // [STAGES][NW][64][LD]
  // [NW][64][CLD], in the ring's place once the last slice is multiplied (the ring is the larger of the two)
  float* cs = reinterpret_cast<float*>(moe_smem);
  static_assert((size_t)NW * MOE_TC_BM * CLD * sizeof(float) <= (size_t)STAGES * (1 + NW) * MOE_TC_BM * LD * sizeof(bf16),
                "the staging tile must fit in the ring");
  __shared__ int src[MOE_TC_BM];
  // (launch_dependents comes at this kernel's end, not its start: it runs in several waves of large blocks,
  // and a successor that starts early would only sit on the SMs its later waves need)
  pdl_wait();
  SB_BEHIND_WAIT(x);
  SB_BEHIND_WAIT(sorted);
  SB_BEHIND_WAIT(tile_expert);
  SB_BEHIND_WAIT(n_tiles);
  const int tile = blockIdx.x;
  if (tile >= n_tiles[0]) return;
  const int e = tile_expert[tile];
  const int n0 = blockIdx.y * MOE_BN;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid < MOE_TC_BM) src[tid] = sorted[tile * MOE_TC_BM + tid];
  __syncthreads();
  const bf16* we = w + (size_t)e * NW * n_out * k_dim;
  // this thread's 16-byte piece of PASSES rows (lm, lm + PASS_ROWS, ..) of every slice
  const int lm = tid / PIECES, lc = (tid % PIECES) * 8;
  const bf16* x_row[PASSES];
  const bf16* w_row[PASSES];
  bool x_in[PASSES], w_in[PASSES];
#pragma unroll
  for (int p = 0; p < PASSES; ++p) {
    const int r = lm + PASS_ROWS * p;
    const int pair = src[r];
    x_in[p] = pair >= 0;
    x_row[p] = x + (UP ? (size_t)(pair >= 0 ? pair / top : 0) : (size_t)tile * MOE_TC_BM + r) * k_dim;
    w_in[p] = n0 + r < n_out;
    w_row[p] = we + (size_t)(w_in[p] ? n0 + r : 0) * k_dim;
  }
  const int k_tiles = (k_dim + BK - 1) / BK;
  auto load = [&](int kt, int st) {
    const int kk = kt * BK + lc;
    const bool in_k = kk < k_dim;
#pragma unroll
    for (int p = 0; p < PASSES; ++p) {
      const int r = lm + PASS_ROWS * p;
      moe_cp16(xs + ((size_t)st * MOE_TC_BM + r) * LD + lc, x_row[p] + (in_k ? kk : 0), in_k && x_in[p]);
#pragma unroll
      for (int a = 0; a < NW; ++a)
        moe_cp16(ws + (((size_t)st * NW + a) * MOE_BN + r) * LD + lc, w_row[p] + (size_t)a * n_out * k_dim + (in_k ? kk : 0),
                 in_k && w_in[p]);
    }
  };
  const int wm = warp & 3, wn = warp >> 2;
  wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[NW][2];
#pragma unroll
  for (int a = 0; a < NW; ++a)
#pragma unroll
    for (int j = 0; j < 2; ++j) wmma::fill_fragment(acc[a][j], 0.f);
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < k_tiles) load(st, st);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();
    const int nk = kt + STAGES - 1;
    if (nk < k_tiles) load(nk, nk % STAGES);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int st = kt % STAGES;
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> fa;
      wmma::load_matrix_sync(fa, xs + ((size_t)st * MOE_TC_BM + wm * 16) * LD + kk, LD);
#pragma unroll
      for (int a = 0; a < NW; ++a)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> fb;
          wmma::load_matrix_sync(fb, ws + (((size_t)st * NW + a) * MOE_BN + wn * 32 + j * 16) * LD + kk, LD);
          wmma::mma_sync(acc[a][j], fa, fb, acc[a][j]);
        }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  pdl_trigger();
  __syncthreads();      // every warp is done with the ring before the staging tile takes its place
#pragma unroll
  for (int a = 0; a < NW; ++a)
#pragma unroll
    for (int j = 0; j < 2; ++j)
      wmma::store_matrix_sync(cs + ((size_t)a * MOE_TC_BM + wm * 16) * CLD + wn * 32 + j * 16, acc[a][j], CLD,
                              wmma::mem_row_major);
  __syncthreads();
  for (int i = tid; i < MOE_TC_BM * MOE_BN; i += 256) {
    const int m = i / MOE_BN, nn = i % MOE_BN;
    const int n = n0 + nn;
    const int row_pair = src[m];
    if (n >= n_out) continue;
    if (MODE == 1) {
      const float g = rnd<bf16>(cs[(size_t)m * CLD + nn]), u = rnd<bf16>(cs[((size_t)(NW - 1) * MOE_TC_BM + m) * CLD + nn]);
      const float a = row_pair >= 0 ? moe_gate(g, u, limit) : 0.f;
      y[((size_t)tile * MOE_TC_BM + m) * n_out + n] = from_f<bf16>(a);
    } else if (MODE == 2) {
      const float u = fmaxf(rnd<bf16>(cs[(size_t)m * CLD + nn]), 0.f);
      y[((size_t)tile * MOE_TC_BM + m) * n_out + n] = from_f<bf16>(row_pair >= 0 ? u * u : 0.f);
    } else if (row_pair >= 0) {
      y[(size_t)row_pair * n_out + n] = from_f<bf16>(cs[(size_t)m * CLD + nn]);
    }
  }
}

// The same for steps with many rows an expert (prompts): tiles of 128 rows times 128 outputs, eight warps
// (two groups of 64 rows times four groups of 32 outputs), mma.sync m16n8k16 with operands by ldmatrix.
// A warp's k-step of 16 is four A loads, two B loads and sixteen products (the 64 x 64 wmma tile above has
// three loads for two products and is bound by them).  Rows and weights arrive in k-slices through a ring of
// three cp.async stages; rows are padded by 16 bytes, so the eight 16-byte rows of an ldmatrix fall into
// eight different bank groups.  The epilogue goes from the accumulators to global memory in pairs.
#define MOE_BIG 128
__device__ __forceinline__ void moe_ldm4(const void* p, uint32_t* r) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void moe_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MODE>
__global__ void __launch_bounds__(256)
moe_tile_big_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                    const int* __restrict__ sorted, const int* __restrict__ tile_expert,
                    const int* __restrict__ n_tiles, int k_dim, int n_out, int top, float limit) {
  constexpr bool UP = MODE != 0;
  // k-slices of 64 (rows of 144 bytes) with one weight block, of 32 (rows of 80 bytes) with two: three stages
  // of either leave room for two blocks an SM
  constexpr int NW = MODE == 1 ? 2 : 1, BK = NW == 1 ? 64 : 32, LD = BK + 8, STAGES = 3;
  constexpr int PIECES = BK / 8, PASS_ROWS = 256 / PIECES, PASSES = MOE_BIG / PASS_ROWS;
  extern __shared__ __align__(128) unsigned char moe_smem[];
  bf16* xs = reinterpret_cast<bf16*>(moe_smem);                          // [STAGES][128][LD]
  bf16* ws = xs + STAGES * MOE_BIG * LD;                                 // [STAGES][NW][128][LD]
  __shared__ int src[MOE_BIG];
  // (launch_dependents comes at this kernel's end, as in the smaller tile: several waves of large blocks)
  pdl_wait();
  SB_BEHIND_WAIT(x);
  SB_BEHIND_WAIT(sorted);
  SB_BEHIND_WAIT(tile_expert);
  SB_BEHIND_WAIT(n_tiles);
  const int tile = blockIdx.x;
  if (tile >= n_tiles[0]) return;
  const int e = tile_expert[tile];
  const int n0 = blockIdx.y * MOE_BIG;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < MOE_BIG) src[tid] = sorted[tile * MOE_BIG + tid];
  __syncthreads();
  const bf16* we = w + (size_t)e * NW * n_out * k_dim;
  // this thread copies one 16-byte piece of PASSES rows (lm, lm + PASS_ROWS, ..) of every slice of rows and of weights
  const int lm = tid / PIECES, lc = (tid % PIECES) * 8;
  const bf16* x_row[PASSES];
  const bf16* w_row[PASSES];
  bool x_in[PASSES], w_in[PASSES];
#pragma unroll
  for (int h = 0; h < PASSES; ++h) {
    const int r = lm + PASS_ROWS * h;
    const int pair = src[r];
    x_in[h] = pair >= 0;
    x_row[h] = x + (UP ? (size_t)(pair >= 0 ? pair / top : 0) : (size_t)tile * MOE_BIG + r) * k_dim;
    w_in[h] = n0 + r < n_out;
    w_row[h] = we + (size_t)(w_in[h] ? n0 + r : 0) * k_dim;
  }
  const int k_tiles = (k_dim + BK - 1) / BK;
  auto load = [&](int kt, int st) {
    const int kk = kt * BK + lc;
    const bool in_k = kk < k_dim;
    const int ko = in_k ? kk : 0;
#pragma unroll
    for (int h = 0; h < PASSES; ++h) {
      const int r = lm + PASS_ROWS * h;
      moe_cp16(xs + ((size_t)st * MOE_BIG + r) * LD + lc, x_row[h] + ko, in_k && x_in[h]);
#pragma unroll
      for (int a = 0; a < NW; ++a)
        moe_cp16(ws + (((size_t)st * NW + a) * MOE_BIG + r) * LD + lc, w_row[h] + (size_t)a * n_out * k_dim + ko,
                 in_k && w_in[h]);
    }
  };
  const int wm = warp & 1, wn = warp >> 1;               // rows 64 wm .., outputs 32 wn ..
  float acc[NW][4][4][4];
#pragma unroll
  for (int a = 0; a < NW; ++a)
#pragma unroll
    for (int mb = 0; mb < 4; ++mb)
#pragma unroll
      for (int nb = 0; nb < 4; ++nb)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][mb][nb][c] = 0.f;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < k_tiles) load(st, st);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  const int a_row = wm * 64 + (lane & 15), a_col = (lane >> 4) * 8;
  const int b_row = wn * 32 + (lane & 7) + (lane >> 4) * 8, b_col = ((lane >> 3) & 1) * 8;
  for (int kt = 0; kt < k_tiles; ++kt) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();
    const int nk = kt + STAGES - 1;
    if (nk < k_tiles) load(nk, nk % STAGES);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const int st = kt % STAGES;
    const bf16* xt = xs + (size_t)st * MOE_BIG * LD;
#pragma unroll
    for (int kk = 0; kk < BK; kk += 16) {
      uint32_t af[4][4];
#pragma unroll
      for (int mb = 0; mb < 4; ++mb) moe_ldm4(xt + (size_t)(a_row + mb * 16) * LD + kk + a_col, af[mb]);
#pragma unroll
      for (int a = 0; a < NW; ++a) {
        const bf16* wt = ws + ((size_t)st * NW + a) * MOE_BIG * LD;
#pragma unroll
        for (int nb2 = 0; nb2 < 2; ++nb2) {
          uint32_t bfr[4];
          moe_ldm4(wt + (size_t)(b_row + nb2 * 16) * LD + kk + b_col, bfr);
#pragma unroll
          for (int mb = 0; mb < 4; ++mb) {
            moe_mma(acc[a][mb][nb2 * 2], af[mb], bfr[0], bfr[1]);
            moe_mma(acc[a][mb][nb2 * 2 + 1], af[mb], bfr[2], bfr[3]);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  pdl_trigger();
  // accumulator (mb, nb, c): row 64 wm + 16 mb + lane / 4 + 8 (c / 2), output 32 wn + 8 nb + 2 (lane % 4) + c % 2;
  // n_out is even here (a multiple of 16), so a pair of outputs is inside or outside together
#pragma unroll
  for (int mb = 0; mb < 4; ++mb)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = wm * 64 + mb * 16 + (lane >> 2) + 8 * h;
      const int row_pair = src[m];
      if (MODE == 0 && row_pair < 0) continue;
      bf16* y_row = y + (MODE == 0 ? (size_t)row_pair : (size_t)tile * MOE_BIG + m) * n_out;
#pragma unroll
      for (int nb = 0; nb < 4; ++nb) {
        const int n = n0 + wn * 32 + nb * 8 + (lane & 3) * 2;
        if (n >= n_out) continue;
        float r0, r1;
        if (MODE == 1) {
          float g0 = rnd<bf16>(acc[0][mb][nb][2 * h]), g1 = rnd<bf16>(acc[0][mb][nb][2 * h + 1]);
          float u0 = rnd<bf16>(acc[NW - 1][mb][nb][2 * h]), u1 = rnd<bf16>(acc[NW - 1][mb][nb][2 * h + 1]);
          r0 = row_pair >= 0 ? moe_gate(g0, u0, limit) : 0.f;
          r1 = row_pair >= 0 ? moe_gate(g1, u1, limit) : 0.f;
        } else if (MODE == 2) {
          const float u0 = fmaxf(rnd<bf16>(acc[0][mb][nb][2 * h]), 0.f), u1 = fmaxf(rnd<bf16>(acc[0][mb][nb][2 * h + 1]), 0.f);
          r0 = row_pair >= 0 ? u0 * u0 : 0.f;
          r1 = row_pair >= 0 ? u1 * u1 : 0.f;
        } else {
          r0 = acc[0][mb][nb][2 * h];
          r1 = acc[0][mb][nb][2 * h + 1];
        }
        *reinterpret_cast<__nv_bfloat162*>(y_row + n) = __floats2bfloat162_rn(r0, r1);
      }
    }
}

// For steps with a handful of rows an expert (single tokens): a tile is up to MOE_FEW rows of one expert, kept
// in shared memory as floats; a block takes MOE_FEW_NB weight rows, a warp one weight row at a time, which its
// lanes read in 16-byte pieces (several in flight) and multiply with every row of the tile; sums in float,
// joined by shuffles.  The weights are read once per tile and nothing is multiplied for padding: the step is
// bound by the weights' bytes, not by tiles of 64 rows of which two are real.
#define MOE_FEW 4
#define MOE_FEW_NB 64
#define MOE_FEW_MAX_K 12800
__device__ __forceinline__ void moe_unpack8(const uint4& v, float* f) {
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}

template <int MODE>
__global__ void __launch_bounds__(256)
moe_few_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
               const int* __restrict__ sorted, const int* __restrict__ tile_expert, const int* __restrict__ n_tiles,
               int k_dim, int n_out, int top, float limit) {
  constexpr bool UP = MODE != 0;
  constexpr int NW = MODE == 1 ? 2 : 1;
  extern __shared__ __align__(16) float moe_xf[];       // [MOE_FEW][k_dim]
  __shared__ int src[MOE_FEW];
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(x);
  SB_BEHIND_WAIT(sorted);
  SB_BEHIND_WAIT(tile_expert);
  SB_BEHIND_WAIT(n_tiles);
  const int tile = blockIdx.x;
  if (tile >= n_tiles[0]) return;
  const int e = tile_expert[tile];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < MOE_FEW) src[tid] = sorted[tile * MOE_FEW + tid];
  __syncthreads();
  int nr = 0;                                            // an expert's pairs fill its tiles from the front
#pragma unroll
  for (int r = 0; r < MOE_FEW; ++r)
    if (src[r] >= 0) nr = r + 1;
  const int chunks = k_dim / 8;
  for (int r = 0; r < nr; ++r) {
    const bf16* xr = x + (UP ? (size_t)(src[r] / top) : (size_t)tile * MOE_FEW + r) * k_dim;
    for (int c = tid; c < chunks; c += 256) {
      float f[8];
      moe_unpack8(*reinterpret_cast<const uint4*>(xr + c * 8), f);
      float4* to = reinterpret_cast<float4*>(moe_xf + (size_t)r * k_dim + c * 8);
      to[0] = make_float4(f[0], f[1], f[2], f[3]);
      to[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
  }
  __syncthreads();
  const bf16* we = w + (size_t)e * NW * n_out * k_dim;
  constexpr int PER_WARP = MOE_FEW_NB / 8;
  const int n_first = blockIdx.y * MOE_FEW_NB + warp * PER_WARP;
  if (n_first >= n_out) return;
  // the warp walks k once: at every piece its PER_WARP weight rows' loads are in flight together, and the
  // tile's rows of that piece are read from shared memory once for all of them
  float acc[NW][PER_WARP][MOE_FEW];
#pragma unroll
  for (int a = 0; a < NW; ++a)
#pragma unroll
    for (int i = 0; i < PER_WARP; ++i)
#pragma unroll
      for (int r = 0; r < MOE_FEW; ++r) acc[a][i][r] = 0.f;
  for (int c = lane; c < chunks; c += 32) {
    float4 xv[MOE_FEW][2];
#pragma unroll
    for (int r = 0; r < MOE_FEW; ++r) {
      if (r < nr) {
        const float4* from = reinterpret_cast<const float4*>(moe_xf + (size_t)r * k_dim + c * 8);
        xv[r][0] = from[0];
        xv[r][1] = from[1];
      } else {
        xv[r][0] = xv[r][1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int a = 0; a < NW; ++a) {
      uint4 wv[PER_WARP];
#pragma unroll
      for (int i = 0; i < PER_WARP; ++i) {
        const int n = min(n_first + i, n_out - 1);       // (a row past the end repeats the last one; it is not stored)
        wv[i] = __ldg(reinterpret_cast<const uint4*>(we + ((size_t)a * n_out + n) * k_dim) + c);
      }
#pragma unroll
      for (int i = 0; i < PER_WARP; ++i) {
        float f[8];
        moe_unpack8(wv[i], f);
#pragma unroll
        for (int r = 0; r < MOE_FEW; ++r) {
          if (r < nr) {
            const float4 p = xv[r][0], q = xv[r][1];
            acc[a][i][r] += f[0] * p.x + f[1] * p.y + f[2] * p.z + f[3] * p.w + f[4] * q.x + f[5] * q.y + f[6] * q.z + f[7] * q.w;
          }
        }
      }
    }
  }
#pragma unroll
  for (int a = 0; a < NW; ++a)
#pragma unroll
    for (int i = 0; i < PER_WARP; ++i)
#pragma unroll
      for (int r = 0; r < MOE_FEW; ++r) acc[a][i][r] = warp_sum(acc[a][i][r]);
  // lane 4 i + r files weight row i for the tile's row r
  float v0 = 0.f, v1 = 0.f;
#pragma unroll
  for (int i = 0; i < PER_WARP; ++i)
#pragma unroll
    for (int r = 0; r < MOE_FEW; ++r)
      if (lane == i * MOE_FEW + r) { v0 = acc[0][i][r]; v1 = acc[NW - 1][i][r]; }
  static_assert(PER_WARP * MOE_FEW == 32, "a lane for every (weight row, tile row)");
  const int n = n_first + lane / MOE_FEW, r = lane % MOE_FEW;
  if (n < n_out && r < nr) {
    if (MODE == 1) {
      y[((size_t)tile * MOE_FEW + r) * n_out + n] = from_f<bf16>(moe_gate(rnd<bf16>(v0), rnd<bf16>(v1), limit));
    } else if (MODE == 2) {
      const float u = fmaxf(rnd<bf16>(v0), 0.f);
      y[((size_t)tile * MOE_FEW + r) * n_out + n] = from_f<bf16>(u * u);
    } else {
      y[(size_t)src[r] * n_out + n] = from_f<bf16>(v0);
    }
  }
}

// The rows of h in the order of `sorted` (a pair's row is h[pair / top]; zeros where a tile is padded), for a
// product that wants its rows in place: a block a row, 16-byte pieces.  Rows behind the last tile stay unwritten.
__global__ void moe_gather_kernel(const bf16* __restrict__ h, const int* __restrict__ sorted,
                                  const int* __restrict__ n_tiles, int tile_rows, int top, bf16* __restrict__ out,
                                  int width) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(h);
  SB_BEHIND_WAIT(sorted);
  SB_BEHIND_WAIT(n_tiles);
  const int row = blockIdx.x;
  if (row >= n_tiles[0] * tile_rows) return;
  const int pair = sorted[row];
  const uint4* from = reinterpret_cast<const uint4*>(h + (size_t)(pair >= 0 ? pair / top : 0) * width);
  uint4* to = reinterpret_cast<uint4*>(out + (size_t)row * width);
  for (int c = threadIdx.x; c < width / 8; c += blockDim.x) to[c] = pair >= 0 ? from[c] : make_uint4(0u, 0u, 0u, 0u);
}

// ids / h (null: every choice is a real expert): a choice from `experts` on stands for the token's own row h[t].
// shared / shared_gate (null: none): shared_gate[t] * shared[t] is added.
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ down, const float* __restrict__ weights, T* __restrict__ out,
                                   int width, int top, const int* __restrict__ ids, int experts, const T* __restrict__ h,
                                   const T* __restrict__ shared, const float* __restrict__ shared_gate) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(down);
  SB_BEHIND_WAIT(weights);
  SB_BEHIND_WAIT(ids);
  SB_BEHIND_WAIT(h);
  SB_BEHIND_WAIT(shared);
  SB_BEHIND_WAIT(shared_gate);
  const int row = blockIdx.x;
  const float sg = shared ? shared_gate[row] : 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < top; ++j) {
      const bool own = ids && ids[(size_t)row * top + j] >= experts;
      a += weights[(size_t)row * top + j] *
           to_f<T>(own ? h[(size_t)row * width + c] : down[((size_t)row * top + j) * width + c]);
    }
    if (shared) a += sg * to_f<T>(shared[(size_t)row * width + c]);
    out[(size_t)row * width + c] = from_f<T>(a);
  }
}

// up 1: x = h [n_tokens, k_dim], w = [experts, 2 * n_out, k_dim] (gate rows, then up rows), y =
// [capacity, n_out] in the order of `sorted`, the clamped gated activation.  up 2: the same with w =
// [experts, n_out, k_dim] and the squared relu.  up 0: x = that y [capacity, k_dim], w = [experts,
// n_out, k_dim], y = [n_pairs, n_out] by pair.
template <int MODE>
static int moe_tiles_mode(int dtype, int tile_rows, const void* x, const void* w, void* y, const int* sorted,
                          const int* tile_expert, const int* n_tiles, int max_tiles, int k_dim, int n_out, int top,
                          float limit, cudaStream_t s) {
  if (tile_rows == MOE_FEW) {
    if (dtype != 1 || k_dim % 8 || k_dim > MOE_FEW_MAX_K || ((uintptr_t)x % 16) || ((uintptr_t)w % 16)) return -2;
    const size_t smem = (size_t)MOE_FEW * k_dim * sizeof(float);
    static size_t configured = 0;
    if (smem > configured) {
      cudaError_t err = cudaFuncSetAttribute(moe_few_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (err != cudaSuccess) return (int)err;
      configured = smem;
    }
    return launch_dependent(moe_few_kernel<MODE>, dim3(max_tiles, (n_out + MOE_FEW_NB - 1) / MOE_FEW_NB), dim3(256), smem, s,
                            (const bf16*)x, (const bf16*)w, (bf16*)y, sorted, tile_expert, n_tiles, k_dim, n_out, top, limit);
  }
  if (tile_rows == MOE_BIG) {
    if (dtype != 1 || k_dim % 16 || n_out % 2 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16) || ((uintptr_t)y % 4)) return -2;
    constexpr int NW = MODE == 1 ? 2 : 1, LD = (NW == 1 ? 64 : 32) + 8;
    const size_t smem = (size_t)3 * (1 + NW) * MOE_BIG * LD * sizeof(bf16);
    cudaFuncSetAttribute(moe_tile_big_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(moe_tile_big_kernel<MODE>, dim3(max_tiles, (n_out + MOE_BIG - 1) / MOE_BIG), dim3(256), smem, s,
                            (const bf16*)x, (const bf16*)w, (bf16*)y, sorted, tile_expert, n_tiles, k_dim, n_out, top, limit);
  }
  const dim3 grid(max_tiles, (n_out + MOE_BN - 1) / MOE_BN);
  if (tile_rows == MOE_TC_BM) {
    if (dtype != 1 || k_dim % 16 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16)) return -2;
    constexpr int NW = MODE == 1 ? 2 : 1;
    const size_t smem = (size_t)3 * (1 + NW) * 64 * (MOE_TC_BK + 8) * sizeof(bf16);
    cudaFuncSetAttribute(moe_tile_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(moe_tile_tc_kernel<MODE>, grid, dim3(256), smem, s, (const bf16*)x, (const bf16*)w,
                            (bf16*)y, sorted, tile_expert, n_tiles, k_dim, n_out, top, limit);
  }
  if (tile_rows != MOE_BM) return -2;
  if (dtype == 0)
    return launch_dependent(moe_tile_kernel<float, MODE>, grid, dim3(256), 0, s, (const float*)x, (const float*)w,
                            (float*)y, sorted, tile_expert, n_tiles, k_dim, n_out, top, limit);
  return launch_dependent(moe_tile_kernel<bf16, MODE>, grid, dim3(256), 0, s, (const bf16*)x, (const bf16*)w,
                          (bf16*)y, sorted, tile_expert, n_tiles, k_dim, n_out, top, limit);
}

extern "C" {

// Rows of a tile for these operands: 64 when both products run on the tensor-core tiles (bfloat16, width and
// inner size multiples of 16), else 32.
int sb_moe_tile_rows(int dtype, int width, int inner) {
  return dtype == 1 && width % 16 == 0 && inner % 16 == 0 ? MOE_TC_BM : MOE_BM;
}
// The same for a step of `n_pairs` (row, expert) pairs over `experts` experts: when the tensor-core tiles take
// the operands, 4 up to four rows an expert on average (the few-row kernel), 128 from 128 rows an expert on average (the large tiles pay for their padding from there
// on) and 256 from 256 (the row tiles of the grouped tcgen05 product, which runs in place of these tiles);
// else as above.
int sb_moe_tile_rows_for(int dtype, int width, int inner, long long n_pairs, int experts) {
  const int rows = sb_moe_tile_rows(dtype, width, inner);
  if (rows != MOE_TC_BM) return rows;
  // 4: the few-row kernel, up to four rows an expert on average (single tokens)
  if (n_pairs <= (long long)MOE_FEW * experts && width <= MOE_FEW_MAX_K && inner <= MOE_FEW_MAX_K) return MOE_FEW;
  // 256: the grouped tcgen05 product (its row tiles), from 256 rows an expert on average
  if (n_pairs >= 256ll * experts) return 256;
  return n_pairs >= (long long)MOE_BIG * experts ? MOE_BIG : rows;
}

// h [.., width] bfloat16 with width a multiple of 8, 16-byte aligned; out [capacity, width].
int sb_moe_gather(const void* h, const int* sorted, const int* n_tiles, int tile_rows, int top, void* out, int capacity,
                  int width, cudaStream_t s) {
  if (capacity == 0) return 0;
  if (width % 8 || ((uintptr_t)h % 16) || ((uintptr_t)out % 16) || top < 1) return -2;
  return launch_dependent(moe_gather_kernel, dim3(capacity), dim3(width / 8 >= 256 ? 256 : 128), 0, s, (const bf16*)h,
                          sorted, n_tiles, tile_rows, top, (bf16*)out, width);
}
int sb_moe_max_experts() { return MOE_MAX_EXPERTS; }
int sb_moe_max_top() { return MOE_MAX_TOP; }

// h: [n_tokens, width]; w: float [experts, width]; b: float [experts] or null; ids: int [n_tokens, top];
// weights: float [n_tokens, top].
// scoring 0: softmax over the chosen logits; 1: sigmoid scores divided by their sum, times weight_scale.
int sb_moe_route(int dtype, const void* h, const float* w, const float* b, int* ids, float* weights, int n_tokens,
                 int width, int experts, int top, int scoring, float weight_scale, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if (experts < 1 || experts > MOE_MAX_EXPERTS || top < 1 || top > MOE_MAX_TOP || top > experts) return -2;
  if (scoring != 0 && scoring != 1) return -2;
  const size_t smem = (size_t)experts * sizeof(float);
  // a step of few rows leaves most SMs idle: a warp an expert (up to 16) shortens the one block a row
  const int threads = n_tokens <= 64 ? (experts >= 16 ? 512 : experts > 4 ? 256 : 128) : 128;
  if (dtype == 0)
    return launch_dependent(moe_route_kernel<float>, dim3(n_tokens), dim3(threads), smem, s, (const float*)h, w, b, ids,
                            weights, width, experts, top, scoring, weight_scale);
  return launch_dependent(moe_route_kernel<bf16>, dim3(n_tokens), dim3(threads), smem, s, (const bf16*)h, w, b, ids,
                          weights, width, experts, top, scoring, weight_scale);
}

int sb_moe_align(const int* ids, int n_pairs, int experts, int* sorted, int capacity, int* tile_expert, int* n_tiles,
                 int tile_rows, cudaStream_t s) {
  if (experts < 1 || experts > MOE_MAX_EXPERTS || tile_rows < 1) return -2;
  return launch_dependent(moe_align_kernel, dim3(1), dim3(256), 0, s, ids, n_pairs, experts, sorted, capacity,
                          tile_expert, n_tiles, tile_rows);
}

int sb_moe_tiles(int dtype, int up, int tile_rows, const void* x, const void* w, void* y, const int* sorted,
                 const int* tile_expert, const int* n_tiles, int max_tiles, int k_dim, int n_out, int top, float limit,
                 cudaStream_t s) {
  if (max_tiles == 0) return 0;
#define MOE_ARGS dtype, tile_rows, x, w, y, sorted, tile_expert, n_tiles, max_tiles, k_dim, n_out, top, limit, s
  if (up == 0) return moe_tiles_mode<0>(MOE_ARGS);
  if (up == 1) return moe_tiles_mode<1>(MOE_ARGS);
  if (up == 2) return moe_tiles_mode<2>(MOE_ARGS);
#undef MOE_ARGS
  return -2;
}

int sb_moe_combine(int dtype, const void* down, const float* weights, void* out, int n_tokens, int width, int top,
                   const int* ids, int experts, const void* h, const void* shared, const float* shared_gate,
                   cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if ((ids != nullptr) != (h != nullptr) || (shared != nullptr) != (shared_gate != nullptr)) return -2;
  const int threads = width >= 1024 ? 256 : 128;
  if (dtype == 0)
    return launch_dependent(moe_combine_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, (const float*)down,
                            weights, (float*)out, width, top, ids, experts, (const float*)h, (const float*)shared,
                            shared_gate);
  return launch_dependent(moe_combine_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, s, (const bf16*)down, weights,
                          (bf16*)out, width, top, ids, experts, (const bf16*)h, (const bf16*)shared, shared_gate);
}

// The router that scores by the softmax over all `outputs` rows of w (float [outputs (+ 1), width]): the choice
// goes by score + correction (float [outputs] or null) among the outputs of the `keep` of `groups` equal groups
// of neighbours whose largest such number is largest (the lower index first among equals, here and in the
// choice); weights: the chosen plain scores over their sum (+ 1e-20), times weight_scale.  gate_out (null:
// none): w has one row more, and gate_out[t] = sigmoid of that row's product.
int sb_moe_route_all(int dtype, const void* h, const float* w, const float* correction, int* ids, float* weights,
                     float* gate_out, int n_tokens, int width, int outputs, int top, int groups, int keep,
                     float weight_scale, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if (outputs < 1 || outputs > MOE_MAX_EXPERTS || top < 1 || top > MOE_MAX_TOP) return -2;
  if (groups < 1 || outputs % groups || keep < 1 || keep > groups || top > outputs / groups * keep) return -2;
  const size_t smem = (size_t)(3 * outputs + 1 + groups) * sizeof(float);
  const int threads = n_tokens <= 64 ? (outputs >= 16 ? 512 : outputs > 4 ? 256 : 128) : 128;
  if (dtype == 0)
    return launch_dependent(moe_route_all_kernel<float>, dim3(n_tokens), dim3(threads), smem, s, (const float*)h, w,
                            correction, ids, weights, gate_out, width, outputs, top, groups, keep, weight_scale);
  return launch_dependent(moe_route_all_kernel<bf16>, dim3(n_tokens), dim3(threads), smem, s, (const bf16*)h, w,
                          correction, ids, weights, gate_out, width, outputs, top, groups, keep, weight_scale);
}

}  // extern "C"
