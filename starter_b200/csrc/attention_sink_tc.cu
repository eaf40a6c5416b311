// The attention of attention_sink.cu on tensor cores (bfloat16): distance penalty, chunks, window, sink
// and head gate as there, for prompts, portions and single tokens alike.
//
// A block takes ONE key/value head and up to 64 query rows that read it: the `group` query heads of that
// key/value head for 64 / group consecutive tokens of a sequence (row r = token r / group, head r % group).
// So a page of keys and values is fetched once for all the query heads that share it, and a single token
// still fills `group` rows of a tile.  Its four warps hold 16 rows each as mma.sync m16n8k16 fragments and
// walk the sequence's pages (64 keys each) from the first key any of its rows may see (the start of the
// first token's chunk or window) to the last token's own position, with the online softmax in float.
// Pages arrive through 16-byte asynchronous copies, two pages ahead of the math, in XOR-swizzled tiles
// (keys [64][dim], values [64][vdim]).
//
// Scores are kept in the base-2 domain: s = q.k * scale * log2(e) - r1 * log2(1 + r2 * (i - j)), since
// ln(x) * log2(e) = log2(x); the sink enters as the state the running softmax starts from (maximum =
// sink * log2(e), sum = 1).  Each row carries its own position, head, sink and gate.  The penalty of a
// page depends on the head and on i - j alone, and a block's rows and a page's keys span at most 127
// distances: the block forms those values once per page and head in shared memory (a table of 128
// entries a head, made while the page before is multiplied) instead of one logarithm per score.  Pages
// that lie wholly inside what every row may see skip the mask; warps without a valid row (a single
// token fills only `group` rows) skip the arithmetic and only help to copy.
//
// A block with at most 16 valid rows (a single token of up to 16 query heads a key/value head) would leave
// three of its four warps idle and the fourth with a page's whole chain of products.  There the warps share
// the KEYS instead: all four hold the same 16 rows, warp w takes keys 16w .. 16w + 15 of every page with a
// running softmax of its own, and the four (maximum, sum, accumulator) are joined through shared memory
// at the end.
//
// With n_splits > 1 the pages of a block are dealt out to gridDim.z blocks, which leave (maximum, sum,
// accumulator) per row in scratch memory for sink_merge_kernel: for steps of few rows (single tokens).
// The sink belongs to the first part alone.
#include "common.cuh"

#define SK_ROWS 64
#define SK_WARPS 4
#define SK_THREADS (SK_WARPS * 32)

__device__ __forceinline__ uint32_t sk_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sk_cp16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sk_smem(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void sk_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void sk_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void sk_ldm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void sk_ldm4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void sk_mma(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sk_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// Byte offset of 16-byte column `chunk` of `row` in a [rows][D] bfloat16 tile with swizzled columns.
template <int D> __device__ __forceinline__ int sk_offset(int row, int chunk) {
  constexpr int C = D / 8;
  const int sw = C >= 8 ? (row & 7) : ((row / (8 / C)) % C);
  return row * D * 2 + ((chunk ^ sw) << 4);
}

template <int D, int DV>
__global__ void __launch_bounds__(SK_THREADS)
sink_attention_tc_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out,
                         float* __restrict__ part_acc, float* __restrict__ part_ml,
                         const bf16* __restrict__ k_store, const bf16* __restrict__ v_store,
                         const int* __restrict__ block_table, int table_stride, const int* __restrict__ seq_slot,
                         const int* __restrict__ seq_q_start, const int* __restrict__ seq_q_len,
                         const int* __restrict__ seq_kv_len, const int* __restrict__ tile_seq,
                         const int* __restrict__ tile_first, const float* __restrict__ r1,
                         const float* __restrict__ r2, const float* __restrict__ sink,
                         const float* __restrict__ gate, int n_tokens, int heads, int kv_heads, int subs,
                         int tokens_per_block, float scale_log2, int chunk, int window) {
  constexpr int CK = D / 8, CV = DV / 8;
  constexpr int K_BYTES = SB_PAGE_TOKENS * D * 2, V_BYTES = SB_PAGE_TOKENS * DV * 2;
  constexpr int KSTEPS = D / 16, NBLK = DV / 8;
  extern __shared__ __align__(128) uint8_t sk_mem[];
  uint8_t* q_tile = sk_mem;                        // [64][D]
  uint8_t* k_tiles = sk_mem + SK_ROWS * D * 2;     // 2 x [64][D]
  uint8_t* v_tiles = k_tiles + 2 * K_BYTES;        // 2 x [64][DV]
  float* pen_tab = reinterpret_cast<float*>(v_tiles + 2 * V_BYTES);   // [group][128], entry tok + 63 - key of the page
  float* pen_coef = pen_tab + (heads / kv_heads) * 128;               // [group][2]: r1 and r2 of the block's heads

  // (no early launch_dependents: the successor starts when this kernel's blocks have exited)
  pdl_wait();
  SB_BEHIND_WAIT(q);
  SB_BEHIND_WAIT(k_store);
  SB_BEHIND_WAIT(v_store);
  SB_BEHIND_WAIT(gate);
  SB_BEHIND_WAIT(seq_q_len);
  SB_BEHIND_WAIT(seq_kv_len);
  SB_BEHIND_WAIT(block_table);
  // key/value heads run fastest: the work list names the tiles with most keys first, and so do the blocks
  const int kvh = blockIdx.x % kv_heads, ts = blockIdx.x / kv_heads;
  const int tile = ts / subs, sub = ts - tile * subs;
  const int split = blockIdx.z, n_splits = gridDim.z;
  const int group = heads / kv_heads;
  const int seq = tile_seq[tile];
  const int q_len = seq_q_len[seq], kv_len = seq_kv_len[seq];
  const int q_first = tile_first[tile] + sub * tokens_per_block;    // first query of this block within the step's tokens of seq
  const int tile_end = min(q_len, tile_first[tile] + SB_PAGE_TOKENS);
  if (q_first >= tile_end) return;
  const int tokens_valid = min(tokens_per_block, tile_end - q_first);
  const int rows_valid = tokens_valid * group;
  const int pos0 = kv_len - q_len + q_first;       // absolute position of the block's first query
  const int* pages = block_table + (size_t)seq_slot[seq] * table_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t tok0 = (size_t)seq_q_start[seq] + q_first;

  const int hi = pos0 + tokens_valid - 1;                                 // last key any row sees
  int lo = 0;                                                             // first key any row sees
  if (chunk > 0) lo = pos0 / chunk * chunk;
  if (window > 0 && pos0 - window + 1 > lo) lo = pos0 - window + 1;
  const int page_lo = lo / SB_PAGE_TOKENS, page_hi = hi / SB_PAGE_TOKENS;
  const int all_tiles = page_hi - page_lo + 1;
  const int per_split = (all_tiles + n_splits - 1) / n_splits;
  const int t_begin = split * per_split, t_end = min(all_tiles, t_begin + per_split);
  const int n_tiles = max(0, t_end - t_begin);

  // ---- stage the queries (rows past the end repeat the last valid row; they are never written)
  for (int idx = tid; idx < SK_ROWS * CK; idx += SK_THREADS) {
    const int r = idx / CK, c = idx % CK;
    const int rr = min(r, rows_valid - 1);
    const bf16* src = q + (tok0 + rr / group) * (size_t)q_stride + (size_t)(kvh * group + rr % group) * D;
    sk_cp16(q_tile + sk_offset<D>(r, c), src + c * 8);
  }
  auto load_kv = [&](int t, int buf) {
    const int page = pages[page_lo + t_begin + t];
    const bf16* ks = k_store + page_row(page, kvh, 0, kv_heads, D);
    const bf16* vs = v_store + page_row(page, kvh, 0, kv_heads, DV);
    for (int idx = tid; idx < SB_PAGE_TOKENS * CK; idx += SK_THREADS)
      sk_cp16(k_tiles + buf * K_BYTES + sk_offset<D>(idx / CK, idx % CK), ks + (size_t)idx * 8);
    for (int idx = tid; idx < SB_PAGE_TOKENS * CV; idx += SK_THREADS)
      sk_cp16(v_tiles + buf * V_BYTES + sk_offset<DV>(idx / CV, idx % CV), vs + (size_t)idx * 8);
  };
  // the penalties of page t: entry [g][x] belongs to the distance pos0 - j0 - 63 + x (negative ones are masked)
  // (thread x forms entry x of every head's table: 128 threads, 128 entries)
  if (r1 && tid < 2 * group) pen_coef[tid] = (tid & 1) ? r2[kvh * group + (tid >> 1)] : r1[kvh * group + (tid >> 1)];
  if (r1) __syncthreads();
  auto make_penalties = [&](int t) {
    if (!r1 || tid >= tokens_valid + 63) return;
    const float d = (float)max(pos0 - (page_lo + t_begin + t) * SB_PAGE_TOKENS - 63 + tid, 0);
    for (int g = 0; g < group; ++g) pen_tab[g * 128 + tid] = pen_coef[2 * g] * __log2f(fmaf(pen_coef[2 * g + 1], d, 1.f));
  };
  if (n_tiles > 0) load_kv(0, 0);
  sk_commit();
  if (n_tiles > 1) load_kv(1, 1);
  sk_commit();
  if (n_tiles > 0) make_penalties(0);
  sk_wait<1>();
  __syncthreads();
  const bool warp_live = rows_valid <= 16 || warp * 16 < rows_valid;
  int lo_last = 0;                                 // the first key the block's last token may see
  if (chunk > 0) lo_last = hi / chunk * chunk;
  if (window > 0 && hi - window + 1 > lo_last) lo_last = hi - window + 1;

  // ---- this warp's 16 query rows as A fragments (with shared keys: every warp the first 16)
  const bool share_keys = rows_valid <= 16;
  const int row_base = share_keys ? 0 : warp * 16;
  uint32_t qf[KSTEPS][4];
  {
    const int r = row_base + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk)
      sk_ldm4(sk_smem(q_tile + sk_offset<D>(r, 2 * kk + (lane >> 4))), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
  }
  // ---- this thread's two rows: where they stand, which head they are, what they may see
  int row_pos[2], row_lo[2], row_head[2], row_pen[2];
  float m_run[2], l_run[2];
  bool row_ok[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_base + (lane >> 2) + 8 * h;
    row_ok[h] = r < rows_valid;
    const int rr = min(r, rows_valid - 1);
    row_pos[h] = pos0 + rr / group;
    row_head[h] = kvh * group + rr % group;
    int first = 0;
    if (chunk > 0) first = row_pos[h] / chunk * chunk;
    if (window > 0 && row_pos[h] - window + 1 > first) first = row_pos[h] - window + 1;
    row_lo[h] = first;
    row_pen[h] = (rr % group) * 128 + rr / group + 63;
    const bool with_sink = sink != nullptr && split == 0 && (!share_keys || warp == 0);
    m_run[h] = with_sink ? sink[row_head[h]] * 1.4426950408889634f : -INFINITY;
    l_run[h] = with_sink && (lane & 3) == 0 ? 1.f : 0.f;      // the row's sum is spread over its four lanes
  }
  float o[NBLK][4];
#pragma unroll
  for (int n = 0; n < NBLK; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    const uint8_t* kt = k_tiles + buf * K_BYTES;
    const uint8_t* vt = v_tiles + buf * V_BYTES;
    const int j0 = (page_lo + t_begin + t) * SB_PAGE_TOKENS;
    if (share_keys) {
      // this warp's 16 keys of the page: S (two blocks of 8 keys), softmax, one k-step of P V
      float s2[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        uint32_t b0, b1, b2, b3;
        const int key = warp * 16 + (lane & 7) + (lane >> 4) * 8;
        sk_ldm4(sk_smem(kt + sk_offset<D>(key, 2 * kk + ((lane >> 3) & 1))), b0, b1, b2, b3);
        sk_mma(s2[0], qf[kk], b0, b1);
        sk_mma(s2[1], qf[kk], b2, b3);
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int h = e >> 1;
          const int jj = warp * 16 + nb * 8 + (lane & 3) * 2 + (e & 1);
          float v = s2[nb][e] * scale_log2;
          if (r1) v -= pen_tab[row_pen[h] - jj];
          if (j0 + jj > row_pos[h] || j0 + jj < row_lo[h]) v = -INFINITY;
          s2[nb][e] = v;
          mx[h] = fmaxf(mx[h], v);
        }
      }
      float alpha[2], m_use[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float m_new = fmaxf(m_run[h], mx[h]);
        m_use[h] = m_new == -INFINITY ? 0.f : m_new;
        alpha[h] = exp2f(m_run[h] - m_use[h]);
        m_run[h] = m_new;
      }
      uint32_t pf1[4];
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        const float p0 = exp2f(s2[nb][0] - m_use[0]), p1 = exp2f(s2[nb][1] - m_use[0]);
        const float p2 = exp2f(s2[nb][2] - m_use[1]), p3 = exp2f(s2[nb][3] - m_use[1]);
        rs[0] += p0 + p1;
        rs[1] += p2 + p3;
        pf1[nb * 2] = sk_pack(p0, p1);
        pf1[nb * 2 + 1] = sk_pack(p2, p3);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + rs[h];
#pragma unroll
      for (int n = 0; n < NBLK; n += 2) {
        o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
        o[n + 1][0] *= alpha[0]; o[n + 1][1] *= alpha[0]; o[n + 1][2] *= alpha[1]; o[n + 1][3] *= alpha[1];
        uint32_t b0, b1, b2, b3;
        const int key = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        sk_ldm4_trans(sk_smem(vt + sk_offset<DV>(key, n + (lane >> 4))), b0, b1, b2, b3);
        sk_mma(o[n], pf1, b0, b1);
        sk_mma(o[n + 1], pf1, b2, b3);
      }
    } else if (warp_live) {
    // S = Q K^T for 64 keys: 8 blocks of 8 keys
    float s[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
      for (int nb = 0; nb < 8; nb += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = nb * 8 + (lane & 7) + (lane >> 4) * 8;
        sk_ldm4(sk_smem(kt + sk_offset<D>(key, 2 * kk + ((lane >> 3) & 1))), b0, b1, b2, b3);
        sk_mma(s[nb], qf[kk], b0, b1);
        sk_mma(s[nb + 1], qf[kk], b2, b3);
      }
    }

    // scale, penalty, mask, online softmax
    const bool edge = j0 + SB_PAGE_TOKENS - 1 > pos0 || j0 < lo_last;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int jj = nb * 8 + (lane & 3) * 2 + (e & 1);
        float v = s[nb][e] * scale_log2;
        if (r1) v -= pen_tab[row_pen[h] - jj];
        if (edge && (j0 + jj > row_pos[h] || j0 + jj < row_lo[h])) v = -INFINITY;
        s[nb][e] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;
      alpha[h] = exp2f(m_run[h] - m_use[h]);
      m_run[h] = m_new;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[4][4];   // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      const float p0 = exp2f(s[nb][0] - m_use[0]), p1 = exp2f(s[nb][1] - m_use[0]);
      const float p2 = exp2f(s[nb][2] - m_use[1]), p3 = exp2f(s[nb][3] - m_use[1]);
      rs[0] += p0 + p1;
      rs[1] += p2 + p3;
      pf[nb >> 1][(nb & 1) * 2] = sk_pack(p0, p1);
      pf[nb >> 1][(nb & 1) * 2 + 1] = sk_pack(p2, p3);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + rs[h];
#pragma unroll
    for (int n = 0; n < NBLK; ++n) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
      o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
    }

    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int n = 0; n < NBLK; n += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        sk_ldm4_trans(sk_smem(vt + sk_offset<DV>(key, n + (lane >> 4))), b0, b1, b2, b3);
        sk_mma(o[n], pf[kk], b0, b1);
        sk_mma(o[n + 1], pf[kk], b2, b3);
      }
    }
    }  // warp_live

    // this buffer and the penalties are free: fetch the tile after next, form the next page's penalties,
    // then make sure the next tile has landed
    __syncthreads();
    if (t + 1 < n_tiles) make_penalties(t + 1);
    if (t + 2 < n_tiles) load_kv(t + 2, buf);
    sk_commit();
    sk_wait<1>();
    __syncthreads();
  }
  sk_wait<0>();

  // ---- finish: a row's sum over its four lanes, then either the head's output or this part's share
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  if (share_keys) {
    // the four warps' shares of the same 16 rows meet in shared memory (the tiles are done with)
    constexpr int LD = DV + 2;                       // a row's accumulator, then its maximum and sum
    float* meet = reinterpret_cast<float*>(sk_mem);  // [4 warps][16 rows][LD]
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float* mine = meet + (size_t)(warp * 16 + (lane >> 2) + 8 * h) * LD;
#pragma unroll
      for (int n = 0; n < NBLK; ++n)
        *reinterpret_cast<float2*>(mine + n * 8 + (lane & 3) * 2) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
      if ((lane & 3) == 0) {
        mine[DV] = m_run[h];
        mine[DV + 1] = l_run[h];
      }
    }
    __syncthreads();
    const size_t n_rows = (size_t)n_tokens * heads;
    for (int idx = tid; idx < rows_valid * DV; idx += SK_THREADS) {
      const int r = idx / DV, c = idx - r * DV;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) M = fmaxf(M, meet[(size_t)(w * 16 + r) * LD + DV]);
      float L = 0.f, a = 0.f;
#pragma unroll
      for (int w = 0; w < SK_WARPS; ++w) {
        const float* theirs = meet + (size_t)(w * 16 + r) * LD;
        const float f = theirs[DV] == -INFINITY ? 0.f : exp2f(theirs[DV] - M);
        L += f * theirs[DV + 1];
        a += f * theirs[c];
      }
      const size_t grow = (tok0 + r / group) * heads + kvh * group + r % group;
      if (n_splits == 1) {
        out[grow * DV + c] = from_f<bf16>(a * (gate ? gate[grow] : 1.f) / L);
      } else {
        part_acc[((size_t)split * n_rows + grow) * DV + c] = a;
        if (c == 0) {
          part_ml[((size_t)split * n_rows + grow) * 2] = M;
          part_ml[((size_t)split * n_rows + grow) * 2 + 1] = L;
        }
      }
    }
    return;
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!row_ok[h]) continue;
    const int r = warp * 16 + (lane >> 2) + 8 * h;
    const size_t token = tok0 + r / group;
    const size_t grow = token * heads + row_head[h];
    if (n_splits == 1) {
      const float f = (gate ? gate[grow] : 1.f) / l_run[h];
      bf16* dst = out + grow * DV;
#pragma unroll
      for (int n = 0; n < NBLK; ++n) {
        const int col = n * 8 + (lane & 3) * 2;
        *reinterpret_cast<uint32_t*>(dst + col) = sk_pack(o[n][2 * h] * f, o[n][2 * h + 1] * f);
      }
    } else {
      const size_t n_rows = (size_t)n_tokens * heads;
      float* pa = part_acc + ((size_t)split * n_rows + grow) * DV;
#pragma unroll
      for (int n = 0; n < NBLK; ++n) {
        const int col = n * 8 + (lane & 3) * 2;
        *reinterpret_cast<float2*>(pa + col) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
      }
      if ((lane & 3) == 0) {
        part_ml[((size_t)split * n_rows + grow) * 2] = m_run[h];
        part_ml[((size_t)split * n_rows + grow) * 2 + 1] = l_run[h];
      }
    }
  }
}

// One warp per (token, head) row: joins the parts' (maximum, sum, accumulator) and applies the gate.
__global__ void sink_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                  const float* __restrict__ gate, bf16* __restrict__ out, int n_rows, int vdim,
                                  int n_splits) {
  pdl_wait();      // no early launch_dependents: the successor starts when this kernel's blocks have exited
  SB_BEHIND_WAIT(part_acc);
  SB_BEHIND_WAIT(part_ml);
  SB_BEHIND_WAIT(gate);
  const int row = (int)(((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_ml[((size_t)s * n_rows + row) * 2]);
  float L = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float m = part_ml[((size_t)s * n_rows + row) * 2];
    if (m != -INFINITY) L += exp2f(m - M) * part_ml[((size_t)s * n_rows + row) * 2 + 1];
  }
  const float f = (gate ? gate[row] : 1.f) / L;
  for (int d = lane; d < vdim; d += 32) {
    float a = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float m = part_ml[((size_t)s * n_rows + row) * 2];
      if (m != -INFINITY) a += exp2f(m - M) * part_acc[((size_t)s * n_rows + row) * vdim + d];
    }
    out[(size_t)row * vdim + d] = from_f<bf16>(a * f);
  }
}

template <int D, int DV>
static int sk_launch(const void* q, int q_stride, void* out, float* part_acc, float* part_ml, const void* k_store,
                     const void* v_store, const int* block_table, int table_stride, const int* seq_slot,
                     const int* seq_q_start, const int* seq_q_len, const int* seq_kv_len, const int* tile_seq,
                     const int* tile_first, int n_tiles, const float* r1, const float* r2, const float* sink,
                     const float* gate, int n_tokens, int heads, int kv_heads, float scale, int chunk, int window,
                     int n_splits, int max_q_len, cudaStream_t s) {
  const int group = heads / kv_heads;
  const int tokens_per_block = SK_ROWS / group;
  int subs = (SB_PAGE_TOKENS + tokens_per_block - 1) / tokens_per_block;
  if (max_q_len > 0) subs = min(subs, (min(max_q_len, SB_PAGE_TOKENS) + tokens_per_block - 1) / tokens_per_block);
  const int smem = SK_ROWS * D * 2 + 2 * SB_PAGE_TOKENS * (D + DV) * 2 + group * 130 * (int)sizeof(float);
  static int configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(sink_attention_tc_kernel<D, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  int rc = launch_dependent(sink_attention_tc_kernel<D, DV>, dim3(n_tiles * subs * kv_heads, 1, n_splits), dim3(SK_THREADS),
                            smem, s, (const bf16*)q, q_stride, (bf16*)out, part_acc, part_ml, (const bf16*)k_store,
                            (const bf16*)v_store, block_table, table_stride, seq_slot, seq_q_start, seq_q_len, seq_kv_len,
                            tile_seq, tile_first, r1, r2, sink, gate, n_tokens, heads, kv_heads, subs, tokens_per_block,
                            scale * 1.4426950408889634f, chunk, window);
  if (rc != 0 || n_splits == 1) return rc;
  const int n_rows = n_tokens * heads;
  return launch_dependent(sink_merge_kernel, dim3((n_rows * 32 + 127) / 128), dim3(128), 0, s, (const float*)part_acc,
                          (const float*)part_ml, gate, (bf16*)out, n_rows, DV, n_splits);
}

extern "C" {

// q: bfloat16 rows of q_stride entries (a multiple of 8, 16-byte aligned) whose first heads * dim are the
// queries; out: [n_tokens, heads * vdim].  The seq_* arrays describe the sequences of the step, tile_seq /
// tile_first its tiles of 64 tokens.  part_acc (float [n_splits, n_tokens * heads, vdim]) and part_ml (float
// [n_splits, n_tokens * heads, 2]) are scratch for n_splits > 1.  dim and vdim: 16, 32, 64 or 128; up to 64
// query heads a key/value head.  max_q_len: the most tokens a sequence brings, if known (fewer idle blocks).
int sb_sink_attention_tc(const void* q, int q_stride, void* out, float* part_acc, float* part_ml, const void* k_store,
                         const void* v_store, const int* block_table, int table_stride, const int* seq_slot,
                         const int* seq_q_start, const int* seq_q_len, const int* seq_kv_len, const int* tile_seq,
                         const int* tile_first, int n_tiles, const float* r1, const float* r2, const float* sink,
                         const float* gate, int n_tokens, int heads, int kv_heads, int dim, int vdim, float scale,
                         int chunk, int window, int n_splits, int max_q_len, cudaStream_t s) {
  if (n_tiles == 0 || n_tokens == 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads || heads / kv_heads > SK_ROWS || n_splits < 1) return -2;
  if ((r1 == nullptr) != (r2 == nullptr) || q_stride % 8 || ((uintptr_t)q % 16)) return -2;
  if (n_splits > 1 && (!part_acc || !part_ml)) return -2;
#define SK_ARGS q, q_stride, out, part_acc, part_ml, k_store, v_store, block_table, table_stride, seq_slot, seq_q_start, \
                seq_q_len, seq_kv_len, tile_seq, tile_first, n_tiles, r1, r2, sink, gate, n_tokens, heads, kv_heads,     \
                scale, chunk, window, n_splits, max_q_len, s
#define SK_BY_V(DD)                                  \
  switch (vdim) {                                    \
    case 16: return sk_launch<DD, 16>(SK_ARGS);      \
    case 32: return sk_launch<DD, 32>(SK_ARGS);      \
    case 64: return sk_launch<DD, 64>(SK_ARGS);      \
    case 128: return sk_launch<DD, 128>(SK_ARGS);    \
    default: return -2;                              \
  }
  switch (dim) {
    case 16: SK_BY_V(16)
    case 32: SK_BY_V(32)
    case 64: SK_BY_V(64)
    case 128: SK_BY_V(128)
    default: return -2;
  }
#undef SK_BY_V
#undef SK_ARGS
}

}  // extern "C"
