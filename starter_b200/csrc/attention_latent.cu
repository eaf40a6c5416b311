// Attention over a cached low-rank latent (multi-head latent attention) with a sliding window.
//
// Per token the cache holds ONE row for all heads: the normed latent c (`rank` entries) followed by a
// rotated key part (`rot` entries) that every head shares.  A head's key is [W_uk c | shared part] and
// its value W_uv c.  Nothing of W_uk and W_uv is applied to the cache here: the caller folds W_uk into
// the query (q' = W_uk^T q_plain, `rank` entries) and applies W_uv to the output, so that
//
//     score(t, s) = (q'_t . c_s + q_rot_t . shared_s) * scale,     o'_t = sum_s softmax(score)_s c_s
//
// and the kernel sees queries of rank + rot entries, keys that are the cache rows and values that are
// their first `rank` entries.  A query at position p sees s with 0 <= p - s < window (window <= 0: all
// s <= p).
//
// latent_prepare: what follows the stacked down-projections of a token.  The query latent is
// RMS-normed (gain qg) into cq; the key/value latent is RMS-normed (gain kg) and filed in the cache
// row of the token's position; the shared key part is turned by the token's position and filed behind
// it.  latent_rotate_q turns the rotated part of every head's query and files it behind q'.
// Rotation: pairs (2i, 2i + 1) of the first rot_dims entries (`split` 0), or pairs (i, i + rot_dims / 2)
// (`split` 1), by the angle whose cos and sin the tables hold at [position][i]; entries from rot_dims on
// pass unchanged.  Norms, angles, scores, the
// softmax and the sums over keys are float.
#include "common.cuh"

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ proj, int proj_width, const float* __restrict__ qg,
                                      const float* __restrict__ kg, float eps, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, int table_width,
                                      const int* __restrict__ tok_pos, const int* __restrict__ tok_slot,
                                      const int* __restrict__ block_table, int table_stride, T* __restrict__ store,
                                      T* __restrict__ cq, int q_rank, int rank, int rot, int rot_dims, int write,
                                      int split) {
  __shared__ float scratch[33];
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(proj);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(tok_slot);
  SB_BEHIND_WAIT(block_table);
  const int row = blockIdx.x;
  const T* pr = proj + (size_t)row * proj_width;
  if (q_rank > 0) {
    float sq = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) {
      const float v = to_f<T>(pr[c]);
      sq += v * v;
    }
    sq = block_sum(sq, scratch);
    const float inv = 1.f / sqrtf(sq / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
      cq[(size_t)row * q_rank + c] = from_f<T>(to_f<T>(pr[c]) * inv * qg[c]);
  }
  if (!write) return;
  const int pos = tok_pos[row];
  const int page = block_table[(size_t)tok_slot[row] * table_stride + pos / SB_PAGE_TOKENS];
  T* dst = store + page_row(page, 0, pos % SB_PAGE_TOKENS, 1, rank + rot);
  const T* kv = pr + q_rank;
  float sq = 0.f;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    const float v = to_f<T>(kv[c]);
    sq += v * v;
  }
  sq = block_sum(sq, scratch);
  const float inv = 1.f / sqrtf(sq / (float)rank + eps);
  for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_f<T>(to_f<T>(kv[c]) * inv * kg[c]);
  const T* shared = kv + rank;
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    const int ia = split ? i : 2 * i, ib = split ? i + rot_dims / 2 : 2 * i + 1;
    const float a = to_f<T>(shared[ia]), b = to_f<T>(shared[ib]);
    const float c = cos_t[(size_t)pos * table_width + i], s = sin_t[(size_t)pos * table_width + i];
    dst[rank + ia] = from_f<T>(a * c - b * s);
    dst[rank + ib] = from_f<T>(b * c + a * s);
  }
  for (int c = rot_dims + threadIdx.x; c < rot; c += blockDim.x) dst[rank + c] = shared[c];
}

// q: [tokens, heads, dim + rot]; qa: [tokens, heads, rank + rot], whose first `rank` entries per head
// the caller fills; this files the turned last `rot` entries of q behind them.
template <typename T>
__global__ void latent_rotate_q_kernel(const T* __restrict__ q, T* __restrict__ qa, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, int table_width,
                                       const int* __restrict__ tok_pos, int heads, int dim, int rot, int rot_dims,
                                       int rank, int split) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(q);
  SB_BEHIND_WAIT(tok_pos);
  const int row = blockIdx.x;
  const int pos = tok_pos[row];
  const int half = rot_dims / 2, rest = rot - rot_dims;
  const int per_head = half + rest;
  for (int e = threadIdx.x; e < heads * per_head; e += blockDim.x) {
    const int h = e / per_head, i = e - h * per_head;
    const T* src = q + ((size_t)row * heads + h) * (dim + rot) + dim;
    T* dst = qa + ((size_t)row * heads + h) * (rank + rot) + rank;
    if (i < half) {
      const int ia = split ? i : 2 * i, ib = split ? i + half : 2 * i + 1;
      const float a = to_f<T>(src[ia]), b = to_f<T>(src[ib]);
      const float c = cos_t[(size_t)pos * table_width + i], s = sin_t[(size_t)pos * table_width + i];
      dst[ia] = from_f<T>(a * c - b * s);
      dst[ib] = from_f<T>(b * c + a * s);
    } else {
      dst[rot_dims + i - half] = src[rot_dims + i - half];
    }
  }
}

// The plain kernel: one warp per (token, head), lanes over the entries of a row; NI = entries a lane.
template <typename T, int NI>
__global__ void latent_attention_kernel(const T* __restrict__ qa, T* __restrict__ out, const T* __restrict__ store,
                                        const int* __restrict__ block_table, int table_stride,
                                        const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                                        int n_tokens, int heads, int rank, int rot, float scale, int window) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(qa);
  SB_BEHIND_WAIT(store);
  SB_BEHIND_WAIT(tok_slot);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(block_table);
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)n_tokens * heads) return;
  const int token = (int)(warp / heads);
  const int width = rank + rot;
  const int pos = tok_pos[token];
  const int* pages = block_table + (size_t)tok_slot[token] * table_stride;
  const T* qr = qa + (size_t)warp * width;
  float qv[NI], acc[NI];
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < width ? to_f<T>(qr[d]) * scale : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  int first = 0;
  if (window > 0 && pos - window + 1 > 0) first = pos - window + 1;
  for (int j0 = first; j0 <= pos; j0 += 4) {
    float s[4];
    float kvv[4][NI];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u;
      s[u] = 0.f;
      if (j <= pos) {
        const T* kr = store + page_row(pages[j / SB_PAGE_TOKENS], 0, j % SB_PAGE_TOKENS, 1, width);
#pragma unroll
        for (int i = 0; i < NI; ++i) {
          const int d = lane + 32 * i;
          kvv[u][i] = d < width ? to_f<T>(kr[d]) : 0.f;
          s[u] += qv[i] * kvv[u][i];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) s[u] = warp_sum(s[u]);
    float m_new = m;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j0 + u <= pos) m_new = fmaxf(m_new, s[u]);
    const float alpha = expf(m - m_new);
    l *= alpha;
#pragma unroll
    for (int i = 0; i < NI; ++i) acc[i] *= alpha;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (j0 + u <= pos) {
        const float p = expf(s[u] - m_new);
        l += p;
#pragma unroll
        for (int i = 0; i < NI; ++i) acc[i] += p * kvv[u][i];
      }
    }
    m = m_new;
  }
  T* orow = out + (size_t)warp * rank;
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int d = lane + 32 * i;
    if (d < rank) orow[d] = from_f<T>(acc[i] * inv);
  }
}

template <typename T>
static int launch_attention(const void* qa, void* out, const void* store, const int* block_table, int table_stride,
                            const int* tok_slot, const int* tok_pos, int n_tokens, int heads, int rank, int rot,
                            float scale, int window, cudaStream_t s) {
  const long long warps = (long long)n_tokens * heads;
  const int threads = 128;
  const dim3 grid((unsigned)((warps * 32 + threads - 1) / threads));
  const int ni = (rank + rot + 31) / 32;
#define GO(N) return launch_dependent(latent_attention_kernel<T, N>, grid, dim3(threads), 0, s, (const T*)qa, (T*)out, \
    (const T*)store, block_table, table_stride, tok_slot, tok_pos, n_tokens, heads, rank, rot, scale, window)
  if (ni <= 2) GO(2);
  if (ni <= 4) GO(4);
  if (ni <= 8) GO(8);
  if (ni <= 12) GO(12);
  if (ni <= 20) GO(20);
#undef GO
  return -2;
}

extern "C" {

int sb_latent_max_row() { return 32 * 20; }

// proj: [n_tokens, proj_width], a row = [query latent (q_rank) | key/value latent (rank) | shared key
// part (rot)] (the query latent alone when write == 0).  cq: [n_tokens, q_rank].  store: one cache
// entry's pages [pages, 1, 64, rank + rot].  cos/sin: float [positions, table_width].
int sb_latent_prepare(int dtype, const void* proj, int proj_width, const float* qg, const float* kg, float eps,
                      const float* cos_t, const float* sin_t, int table_width, const int* tok_pos,
                      const int* tok_slot, const int* block_table, int table_stride, void* store, void* cq,
                      int n_tokens, int q_rank, int rank, int rot, int rot_dims, int write, int split, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if (rot_dims % 2 || rot_dims > rot || rot_dims / 2 > table_width) return -2;
  if (proj_width < q_rank + (write ? rank + rot : 0)) return -2;
  if (dtype == 0)
    return launch_dependent(latent_prepare_kernel<float>, dim3(n_tokens), dim3(128), 0, s, (const float*)proj,
                            proj_width, qg, kg, eps, cos_t, sin_t, table_width, tok_pos, tok_slot, block_table,
                            table_stride, (float*)store, (float*)cq, q_rank, rank, rot, rot_dims, write, split);
  return launch_dependent(latent_prepare_kernel<bf16>, dim3(n_tokens), dim3(128), 0, s, (const bf16*)proj, proj_width,
                          qg, kg, eps, cos_t, sin_t, table_width, tok_pos, tok_slot, block_table, table_stride,
                          (bf16*)store, (bf16*)cq, q_rank, rank, rot, rot_dims, write, split);
}

int sb_latent_rotate_q(int dtype, const void* q, void* qa, const float* cos_t, const float* sin_t, int table_width,
                       const int* tok_pos, int n_tokens, int heads, int dim, int rot, int rot_dims, int rank,
                       int split, cudaStream_t s) {
  if (n_tokens == 0 || rot == 0) return 0;
  if (rot_dims % 2 || rot_dims > rot || rot_dims / 2 > table_width) return -2;
  if (dtype == 0)
    return launch_dependent(latent_rotate_q_kernel<float>, dim3(n_tokens), dim3(128), 0, s, (const float*)q,
                            (float*)qa, cos_t, sin_t, table_width, tok_pos, heads, dim, rot, rot_dims, rank, split);
  return launch_dependent(latent_rotate_q_kernel<bf16>, dim3(n_tokens), dim3(128), 0, s, (const bf16*)q, (bf16*)qa,
                          cos_t, sin_t, table_width, tok_pos, heads, dim, rot, rot_dims, rank, split);
}

// qa: [n_tokens, heads, rank + rot]; out: [n_tokens, heads, rank]; store as above.
int sb_latent_attention(int dtype, const void* qa, void* out, const void* store, const int* block_table,
                        int table_stride, const int* tok_slot, const int* tok_pos, int n_tokens, int heads, int rank,
                        int rot, float scale, int window, cudaStream_t s) {
  if (n_tokens == 0) return 0;
  if (dtype == 0)
    return launch_attention<float>(qa, out, store, block_table, table_stride, tok_slot, tok_pos, n_tokens, heads,
                                   rank, rot, scale, window, s);
  return launch_attention<bf16>(qa, out, store, block_table, table_stride, tok_slot, tok_pos, n_tokens, heads, rank,
                                rot, scale, window, s);
}

}  // extern "C"

// ---------------------------------------------------------------------------------- tensor cores
// The same attention for bfloat16 on mma.sync tiles (rank and rot multiples of 16).  A block owns up to
// 64 query rows: the heads (up to 64 of them) of consecutive tokens of one sequence, which all score the
// same cache rows.  It walks the keys its tokens can see in blocks of 32 (a block of keys never leaves a
// page), double-buffered by cp.async; eight warps = four groups of 16 query rows times two halves.  A warp
// forms the scores S = Q K^T of its half of the block's keys (16 x 16, float), masks them by each row's own
// position and window, and meets the other half through shared memory (the halves' row maxima, then the
// weights P in bfloat16) behind a named barrier of the pair; each half keeps the running maximum, the sum of
// its own keys' weights (the sums meet at the end), and adds P V for its half of the latent's columns, V
// being the first `rank` entries of the very key rows in shared memory.
// With n_splits > 1 the key blocks are dealt out to gridDim.y blocks, which leave (maximum, sum,
// unnormalised sums) per row in scratch memory for latent_merge_kernel: single tokens of few sequences.
#define LA_BM 64
#define LA_BN 32
#define LA_PLD 40      // a row of P: 32 keys and 8 entries of padding (ldmatrix without bank conflicts)

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool real) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int bytes = real ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm4_t(unsigned (&r)[4], const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&p);
}

// The two warps of a row group meet (named barriers 1 to 4; 0 is the block's).
__device__ __forceinline__ void pair_sync(int row_group) {
  asm volatile("bar.sync %0, 64;" ::"r"(row_group + 1) : "memory");
}

template <int NT>   // 8-column tiles of the latent a warp sums (its half of the value columns, rounded up)
__global__ void __launch_bounds__(256, 1)
latent_attention_tc_kernel(const bf16* __restrict__ qa, bf16* __restrict__ out, float* __restrict__ part_acc,
                           float* __restrict__ part_ml, const bf16* __restrict__ store,
                           const int* __restrict__ block_table, int table_stride, const int* __restrict__ seq_slot,
                           const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                           const int* __restrict__ seq_kv_len, const int* __restrict__ tile_seq,
                           const int* __restrict__ tile_first, int heads, int rank, int rot, float scale, int window,
                           int tokens_per_block, int heads_per_block, int head_chunks, int subs, int n_rows_total) {
  extern __shared__ __align__(16) unsigned char latent_smem[];
  const int Dk = rank + rot, ld = Dk + 8;
  bf16* qs = reinterpret_cast<bf16*>(latent_smem);
  bf16* ks = qs + LA_BM * ld;
  bf16* ps = ks + 2 * LA_BN * ld;                                 // [4 row groups][16 rows][LA_PLD]: the weights P
  float* xm = reinterpret_cast<float*>(ps + 4 * 16 * LA_PLD);     // [4 row groups][2 halves][16 rows]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int per_tile = subs * head_chunks;
  const int tile = blockIdx.x / per_tile, rem = blockIdx.x % per_tile;
  const int sub = rem / head_chunks, hc = rem % head_chunks;
  const int split = blockIdx.y, n_splits = gridDim.y;
  // (launch_dependents comes at this kernel's end, not its start: it runs in several waves of large blocks,
  // and a successor that starts early would only sit on the SMs its later waves need)
  pdl_wait();
  SB_BEHIND_WAIT(qa); SB_BEHIND_WAIT(store); SB_BEHIND_WAIT(block_table);
  SB_BEHIND_WAIT(seq_slot); SB_BEHIND_WAIT(seq_q_start); SB_BEHIND_WAIT(seq_q_len); SB_BEHIND_WAIT(seq_kv_len);
  SB_BEHIND_WAIT(tile_seq); SB_BEHIND_WAIT(tile_first);
  const int seq = tile_seq[tile];
  const int q_len = seq_q_len[seq];
  const int first_tok = tile_first[tile] + sub * tokens_per_block;
  if (sub * tokens_per_block >= 64 || first_tok >= q_len) return;
  int n_tok = min(tokens_per_block, q_len - first_tok);
  n_tok = min(n_tok, 64 - sub * tokens_per_block);
  const int h0 = hc * heads_per_block;
  const int n_heads = min(heads_per_block, heads - h0);
  const int kv_len = seq_kv_len[seq], q_start = seq_q_start[seq];
  const int* pages = block_table + (size_t)seq_slot[seq] * table_stride;
  const int p_first = kv_len - q_len + first_tok, p_last = p_first + n_tok - 1;
  const int j_lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int b_lo = j_lo / LA_BN, n_blocks = p_last / LA_BN - b_lo + 1;
  const int per_split = (n_blocks + n_splits - 1) / n_splits;
  const int b_begin = b_lo + split * per_split, b_end = min(b_lo + n_blocks, b_begin + per_split);
  const int chunks = Dk / 8;                      // 16-byte pieces of a row

  // A thread's pieces of a key block: piece tid + 256 k is piece c of row kr, found once here and stepped by
  // k; a block of 32 keys lies in one page, whose number is looked up once a block.
  static_assert(SB_PAGE_TOKENS % LA_BN == 0, "a block of keys must not leave a page");
  const int kr0 = tid / chunks, c0 = tid - kr0 * chunks;
  const int step_r = 256 / chunks, step_c = 256 - step_r * chunks;
  auto load_keys = [&](int b, int buf) {
    bf16* dst = ks + (size_t)buf * LA_BN * ld;
    const int j0 = b * LA_BN;
    const bf16* src0 = store + ((size_t)pages[j0 / SB_PAGE_TOKENS] * SB_PAGE_TOKENS + j0 % SB_PAGE_TOKENS) * Dk;
    int kr = kr0, c = c0;
    while (kr < LA_BN) {
      const bool real = j0 + kr <= p_last;
      const int rr = real ? kr : p_last - j0;       // (a key of the same block stands in; nothing is copied)
      cp_async16(dst + kr * ld + c * 8, src0 + (size_t)rr * Dk + c * 8, real);
      kr += step_r;
      c += step_c;
      if (c >= chunks) { c -= chunks; ++kr; }
    }
  };
  // the queries, and the first block of keys
  for (int i = tid; i < LA_BM * chunks; i += 256) {
    const int r = i / chunks, c = i - r * chunks;
    const int tt = r / heads_per_block, hh = r - tt * heads_per_block;
    const bool real = tt < n_tok && hh < n_heads;
    const bf16* src = qa + ((size_t)(q_start + first_tok + (real ? tt : 0)) * heads + h0 + (real ? hh : 0)) * Dk + c * 8;
    cp_async16(qs + r * ld + c * 8, src, real);
  }
  if (b_begin < b_end) load_keys(b_begin, 0);
  cp_async_commit();

  // neighbouring warps are the two halves of a row group, so that the row groups of a block with few rows
  // (single tokens: `heads` rows of 64) sit on different schedulers
  const int wr = warp >> 1, wc = warp & 1;
  const int g = lane >> 2, tq = lane & 3;
  const int c_half = (rank / 2 + 15) / 16 * 16;
  const int col_lo = wc == 0 ? 0 : c_half, col_hi = wc == 0 ? c_half : rank;
  const int n_pairs = (col_hi - col_lo) / 16;     // pairs of 8-column tiles this warp sums
  int row_pos[2], row_lo[2];
  bool row_ok[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = 16 * wr + g + 8 * i;
    const int tt = r / heads_per_block, hh = r - tt * heads_per_block;
    row_ok[i] = tt < n_tok && hh < n_heads;
    row_pos[i] = p_first + tt;
    row_lo[i] = window > 0 ? row_pos[i] - window + 1 : 0;
  }
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const bool warp_has_rows = __any_sync(0xffffffffu, row_ok[0] || row_ok[1]);   // else: loads and barriers only

  for (int b = b_begin; b < b_end; ++b) {
    const int buf = (b - b_begin) & 1;
    if (b + 1 < b_end) load_keys(b + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const bf16* kb = ks + (size_t)buf * LA_BN * ld;
    if (warp_has_rows) {
    // this warp's half of the block's keys: S = Q K^T for 16 rows x 16 keys
    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    for (int kk = 0; kk < Dk / 16; ++kk) {
      unsigned a[4], kf[4];
      ldsm4(a, qs + (16 * wr + (lane & 15)) * ld + kk * 16 + (lane >> 4) * 8);
      const int mi = lane >> 3;
      ldsm4(kf, kb + (16 * wc + (lane & 7) + (mi >> 1) * 8) * ld + kk * 16 + (mi & 1) * 8);
      mma16816(s[0], a, kf[0], kf[1]);
      mma16816(s[1], a, kf[2], kf[3]);
    }
    // mask by each row's own position and window; the maximum of the half, then of both halves
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = e >> 1;
        const int j = b * LA_BN + 16 * wc + n * 8 + 2 * tq + (e & 1);
        const bool seen = row_ok[i] && j >= row_lo[i] && j <= row_pos[i];
        s[n][e] = seen ? s[n][e] * scale : -INFINITY;
        mx[i] = fmaxf(mx[i], s[n][e]);
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      if (tq == 0) xm[(wr * 2 + wc) * 16 + g + 8 * i] = mx[i];
    }
    pair_sync(wr);
    float alpha[2], m_use[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float m_new = fmaxf(m_run[i], fmaxf(mx[i], xm[(wr * 2 + (wc ^ 1)) * 16 + g + 8 * i]));
      m_use[i] = m_new == -INFINITY ? 0.f : m_new;
      alpha[i] = expf(m_run[i] - m_use[i]);
      m_run[i] = m_new;
      l_run[i] *= alpha[i];
    }
    // the half's weights: summed here (the halves' sums meet at the end), and left for both halves' P V
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        s[n][e] = expf(s[n][e] - m_use[e >> 1]);
        l_run[e >> 1] += s[n][e];
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
        *reinterpret_cast<unsigned*>(ps + (wr * 16 + g + 8 * i) * LA_PLD + 16 * wc + n * 8 + 2 * tq) =
            pack_bf16(s[n][2 * i], s[n][2 * i + 1]);
    }
    pair_sync(wr);
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {   // (no row's maximum moved: nothing to rescale)
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
        o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
      }
    }
#pragma unroll
    for (int k2 = 0; k2 < 2; ++k2) {
      unsigned pa[4];
      ldsm4(pa, ps + (wr * 16 + (lane & 15)) * LA_PLD + k2 * 16 + (lane >> 4) * 8);
      const bf16* v_at = kb + (16 * k2 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + col_lo + (lane >> 4) * 8;
      if (n_pairs == NT / 2) {
        // every tile of the template's count is real (the usual case): no branch between the tiles, so that
        // the loads of the tiles ahead are in flight while a tile multiplies
#pragma unroll
        for (int pr = 0; pr < NT / 2; ++pr) {
          unsigned vf[4];
          ldsm4_t(vf, v_at + pr * 16);
          mma16816(o[2 * pr], pa, vf[0], vf[1]);
          mma16816(o[2 * pr + 1], pa, vf[2], vf[3]);
        }
      } else {
#pragma unroll
        for (int pr = 0; pr < NT / 2; ++pr) {
          if (pr < n_pairs) {
            unsigned vf[4];
            ldsm4_t(vf, v_at + pr * 16);
            mma16816(o[2 * pr], pa, vf[0], vf[1]);
            mma16816(o[2 * pr + 1], pa, vf[2], vf[3]);
          }
        }
      }
    }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  pdl_trigger();
  if (warp_has_rows) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
      l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
      if (tq == 0) xm[(wr * 2 + wc) * 16 + g + 8 * i] = l_run[i];
    }
    pair_sync(wr);
#pragma unroll
    for (int i = 0; i < 2; ++i) l_run[i] += xm[(wr * 2 + (wc ^ 1)) * 16 + g + 8 * i];
  }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (!row_ok[i]) continue;
    const int r = 16 * wr + g + 8 * i;
    const int tt = r / heads_per_block, hh = r - tt * heads_per_block;
    const size_t grow = (size_t)(q_start + first_tok + tt) * heads + h0 + hh;
    if (n_splits == 1) {
      const float inv = 1.f / l_run[i];
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int col = col_lo + n * 8 + 2 * tq;
        if (n < 2 * n_pairs)
          *reinterpret_cast<unsigned*>(out + grow * rank + col) = pack_bf16(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
      }
    } else {
      float* pa = part_acc + ((size_t)split * n_rows_total + grow) * rank;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int col = col_lo + n * 8 + 2 * tq;
        if (n < 2 * n_pairs) *reinterpret_cast<float2*>(pa + col) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
      }
      if (wc == 0 && tq == 0) {
        part_ml[((size_t)split * n_rows_total + grow) * 2] = m_run[i];
        part_ml[((size_t)split * n_rows_total + grow) * 2 + 1] = l_run[i];
      }
    }
  }
}

// out[row] = sum_s acc[s][row] exp(m_s - M) / sum_s l_s exp(m_s - M): a block a row.  The first warp forms
// the parts' factors (a lane a part, up to 32 parts) and leaves them in shared memory; the sums over the
// parts then run without a branch, their loads independent of one another.
__global__ void latent_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                    bf16* __restrict__ out, int n_rows, int rank, int n_splits) {
  __shared__ float factor[32];
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(part_acc);
  SB_BEHIND_WAIT(part_ml);
  const int row = blockIdx.x;
  if (threadIdx.x < 32) {
    const int s = threadIdx.x;
    const bool has = s < n_splits;
    const float m = has ? part_ml[((size_t)s * n_rows + row) * 2] : -INFINITY;
    const float l = has ? part_ml[((size_t)s * n_rows + row) * 2 + 1] : 0.f;
    float M = m;
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float e = m == -INFINITY ? 0.f : expf(m - M);
    float L = l * e;
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    factor[s] = e / L;
  }
  __syncthreads();
  const float* acc = part_acc + (size_t)row * rank;
  const size_t part_stride = (size_t)n_rows * rank;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float a = 0.f;
#pragma unroll 8
    for (int s = 0; s < n_splits; ++s) {
      const float f = factor[s];
      const float v = acc[s * part_stride + c];
      a += f != 0.f ? v * f : 0.f;          // (a part without keys left zeros; its factor is zero)
    }
    out[(size_t)row * rank + c] = from_f<bf16>(a);
  }
}

extern "C" {

// The bfloat16 attention on tensor cores.  seq_* describe the sequences of the step (slot, first packed
// row, rows brought, length with them), tile_seq / tile_first list its tiles of 64 tokens.  part_acc
// (float [n_splits, n_tokens * heads, rank]) and part_ml (float [n_splits, n_tokens * heads, 2]) are
// scratch for n_splits > 1.  max_q_len: the most tokens a sequence brings, if the caller knows (it saves
// launching blocks that would find nothing to do).  Returns -2 for sizes it does not take: rank and rot multiples of 16, rank up
// to 512, rows of up to 640 entries.
int sb_latent_attention_tc(const void* qa, void* out, float* part_acc, float* part_ml, const void* store,
                           const int* block_table, int table_stride, const int* seq_slot, const int* seq_q_start,
                           const int* seq_q_len, const int* seq_kv_len, const int* tile_seq, const int* tile_first,
                           int n_tiles, int n_tokens, int heads, int rank, int rot, float scale, int window, int n_splits,
                           int max_q_len, cudaStream_t s) {
  if (n_tiles == 0 || n_tokens == 0) return 0;
  if (rank % 16 || rot % 16 || rank < 16 || rank > 512 || rank + rot > 640 || n_splits < 1 || n_splits > 32) return -2;
  const int heads_per_block = heads < 64 ? heads : 64;
  const int tokens_per_block = 64 / heads_per_block;
  const int head_chunks = (heads + heads_per_block - 1) / heads_per_block;
  // blocks a tile of 64 tokens is cut into; no sequence brings more than max_q_len (<= 0: unknown)
  const int tile_tokens = max_q_len > 0 && max_q_len < 64 ? max_q_len : 64;
  const int subs = (tile_tokens + tokens_per_block - 1) / tokens_per_block;
  const int ld = rank + rot + 8;
  const size_t smem = (size_t)(LA_BM + 2 * LA_BN) * ld * sizeof(bf16) + 4 * 16 * LA_PLD * sizeof(bf16) + 4 * 2 * 16 * sizeof(float);
  const dim3 grid(n_tiles * subs * head_chunks, n_splits);
  const int c_half = (rank / 2 + 15) / 16 * 16;
  const int nt = c_half / 8;
#define GO(N)                                                                                                         \
  {                                                                                                                   \
    cudaFuncSetAttribute(latent_attention_tc_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
    int rc = launch_dependent(latent_attention_tc_kernel<N>, grid, dim3(256), smem, s, (const bf16*)qa, (bf16*)out,   \
                              part_acc, part_ml, (const bf16*)store, block_table, table_stride, seq_slot, seq_q_start, \
                              seq_q_len, seq_kv_len, tile_seq, tile_first, heads, rank, rot, scale, window,           \
                              tokens_per_block, heads_per_block, head_chunks, subs, n_tokens * heads);                \
    if (rc != 0 || n_splits == 1) return rc;                                                                          \
  }
  if (nt <= 4) GO(4)
  else if (nt <= 8) GO(8)
  else if (nt <= 16) GO(16)
  else GO(32)
#undef GO
  return launch_dependent(latent_merge_kernel, dim3(n_tokens * heads), dim3(128), 0, s, (const float*)part_acc,
                          (const float*)part_ml, (bf16*)out, n_tokens * heads, rank, n_splits);
}

}  // extern "C"
