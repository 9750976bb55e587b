// Paged attention with mma.sync for bfloat16 and head sizes 64 and 128: a tiled kernel for steps
// that hold portions of prompts (any mix of query lengths), two kernels for decode steps (one
// query token per request, split along the keys): one that reads keys straight from global
// memory into mma fragments and values through a per-warp cp.async ring, and one for head size
// 128 that has whole pages brought in by TMA; the end of a decode block that both share (join
// of the warps, then output, scratch, or the join of a cluster over distributed shared memory);
// and the kernel that joins splits left in scratch.
//
// All walk a request's keys through its block table in tiles of 64 keys, compute S = Q K^T with
// mma.sync.m16n8k16 (bf16 in, fp32 out), keep the running maximum and sum of the softmax in fp32
// registers (base-2 exponent with the scale folded in) and accumulate O += P V in fp32.  The
// rows of a tile are (query token, query head) pairs of one kv head: the heads of a group share
// every key tile they read, whatever the group size (7 for Qwen2-7B).  A query at position p
// sees keys max(0, p - window + 1) .. p; keys behind the window may lie on pages that were given
// back (table entry -1) and are never fetched.
//
// Replaces the reference's per-sequence gather + SDPA (src/turboserve/engine/model/
// attention.py:184-209) and its Triton decode kernel (src/turboserve/engine/model/
// triton_attention.py:72-174), which has no tensor cores and no split over the keys.
#include <cuda.h>

#include "common.cuh"

#define TILE_N 64
#define FLASH_WARPS 4
#define FLASH_THREADS (FLASH_WARPS * 32)
#ifndef DECODE_STAGES
#define DECODE_STAGES 5  // value tiles (16 keys, 4 KB at head size 128) in each decode warp's ring
#endif

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ unsigned smem_u32(const void* p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async16(unsigned dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

// byte offset of 16-byte chunk c of key row r inside a [TILE_N][D] bf16 tile
template <int D> __device__ __forceinline__ unsigned tile_offset(int r, int c) {
  return (unsigned)(r * D * 2 + (((c & ~7) | ((c ^ r) & 7)) << 4));
}

// Stage keys key0 .. key0+63 of one kv head into shared memory; keys outside [begin, end) and
// keys whose page is gone are zero-filled.
template <int D>
__device__ __forceinline__ void load_kv_tile(bf16* k_s, bf16* v_s, const bf16* __restrict__ k_pages,
                                             const bf16* __restrict__ v_pages,
                                             const int* __restrict__ table, int key0, int begin,
                                             int end, int page_shift, int num_kv_heads, int kv_head) {
  constexpr int CH = D / 8;
  const unsigned k_base = smem_u32(k_s), v_base = smem_u32(v_s);
  const int page_mask = (1 << page_shift) - 1;
#pragma unroll
  for (int idx = threadIdx.x; idx < TILE_N * CH; idx += FLASH_THREADS) {
    const int r = idx / CH, c = idx % CH;
    const int key = key0 + r;
    bool ok = key >= begin && key < end;
    int page = ok ? table[key >> page_shift] : -1;
    ok = ok && page >= 0;
    const size_t off = ok ? ((((size_t)page << page_shift) + (key & page_mask)) * num_kv_heads + kv_head) * D + c * 8 : 0;
    const unsigned o = tile_offset<D>(r, c);
    cp_async16(k_base + o, k_pages + off, ok ? 16 : 0);
    cp_async16(v_base + o, v_pages + off, ok ? 16 : 0);
  }
}

// ---------------------------------------------------------------------------------------------
// Q fragments of a warp's 16 rows, loaded from global memory (zeros for rows without a query).
// ---------------------------------------------------------------------------------------------
template <int D>
__device__ __forceinline__ void load_q_frags(unsigned (&qf)[D / 16][4], const bf16* row_lo,
                                             const bf16* row_hi, int t) {
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int k = kk * 16 + 2 * t;
    qf[kk][0] = row_lo ? *reinterpret_cast<const unsigned*>(row_lo + k) : 0u;
    qf[kk][1] = row_hi ? *reinterpret_cast<const unsigned*>(row_hi + k) : 0u;
    qf[kk][2] = row_lo ? *reinterpret_cast<const unsigned*>(row_lo + k + 8) : 0u;
    qf[kk][3] = row_hi ? *reinterpret_cast<const unsigned*>(row_hi + k + 8) : 0u;
  }
}

// One warp: S[16 x 8*NT] = Q K^T over the key rows key_row0.. of the staged tile.
template <int D, int NT>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const unsigned (&qf)[D / 16][4],
                                        const bf16* k_s, int key_row0, int lane) {
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[i][e] = 0.0f;
  const unsigned base = smem_u32(k_s);
  const int mi = lane >> 3, lr = lane & 7;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      unsigned b[4];
      const int r = key_row0 + np * 16 + (mi >> 1) * 8 + lr;
      ldmatrix_x4(b, base + tile_offset<D>(r, kk * 2 + (mi & 1)));
      mma16816(s[2 * np], qf[kk], b[0], b[1]);
      mma16816(s[2 * np + 1], qf[kk], b[2], b[3]);
    }
  }
}

// One warp: O[16 x D] += P[16 x 8*NT] V over the key rows key_row0.. of the staged tile.
template <int D, int NT>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const float (&p)[NT][4],
                                        const bf16* v_s, int key_row0, int lane) {
  const unsigned base = smem_u32(v_s);
  const int mi = lane >> 3, lr = lane & 7;
#pragma unroll
  for (int j = 0; j < NT / 2; ++j) {
    unsigned a[4];
    a[0] = pack_bf16(p[2 * j][0], p[2 * j][1]);
    a[1] = pack_bf16(p[2 * j][2], p[2 * j][3]);
    a[2] = pack_bf16(p[2 * j + 1][0], p[2 * j + 1][1]);
    a[3] = pack_bf16(p[2 * j + 1][2], p[2 * j + 1][3]);
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      unsigned b[4];
      const int r = key_row0 + j * 16 + (mi & 1) * 8 + lr;
      ldmatrix_x4_trans(b, base + tile_offset<D>(r, np * 2 + (mi >> 1)));
      mma16816(o[2 * np], a, b[0], b[1]);
      mma16816(o[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// Mask, running maximum, exponentials and running sum for a warp's score tile.  Row "lo" is
// the thread's row g, row "hi" its row g + 8; pos < 0 marks a row without a query.
template <int D, int NT>
__device__ __forceinline__ void softmax_tile(float (&s)[NT][4], float (&o)[D / 8][4], float (&m)[2],
                                             float (&l)[2], int key0, int t, const int (&pos)[2],
                                             const int (&first)[2], float scale_log2) {
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int h = e >> 1;
      const int key = key0 + i * 8 + 2 * t + (e & 1);
      const bool visible = key <= pos[h] && key >= first[h];
      const float v = visible ? s[i][e] * scale_log2 : -INFINITY;
      s[i][e] = v;
      mx[h] = fmaxf(mx[h], v);
    }
  float corr[2], base[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    const float m_new = fmaxf(m[h], mx[h]);
    base[h] = m_new == -INFINITY ? 0.0f : m_new;
    corr[h] = exp2f(m[h] - base[h]);
    m[h] = m_new;
    l[h] *= corr[h];
  }
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float pv = exp2f(s[i][e] - base[e >> 1]);
      s[i][e] = pv;
      l[e >> 1] += pv;
    }
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    o[i][0] *= corr[0]; o[i][1] *= corr[0];
    o[i][2] *= corr[1]; o[i][3] *= corr[1];
  }
}

// The same step for the tiled kernel, with fewer instructions per score: the running maximum
// is kept in raw score units (the scale is positive, so the order is the same) and the
// exponential is one fused multiply-add and one ex2 per score; a tile that every row of the
// warp sees in full (MASKED == false: below the diagonal and inside the window) skips the
// visibility tests.  Rows without a query have zero queries: their arithmetic stays finite and
// their results are never stored.
template <int D, int NT, bool MASKED>
__device__ __forceinline__ void softmax_tile_raw(float (&s)[NT][4], float (&o)[D / 8][4], float (&m)[2],
                                                 float (&l)[2], int key0, int t, const int (&pos)[2],
                                                 const int (&first)[2], float scale_log2) {
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int h = e >> 1;
      if (MASKED) {
        const int key = key0 + i * 8 + 2 * t + (e & 1);
        if (!(key <= pos[h] && key >= first[h])) s[i][e] = -INFINITY;
      }
      mx[h] = fmaxf(mx[h], s[i][e]);
    }
  float corr[2], shift[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
    mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    const float m_new = fmaxf(m[h], mx[h]);
    const float base = m_new == -INFINITY ? 0.0f : m_new;
    corr[h] = exp2f((m[h] - base) * scale_log2);
    shift[h] = -base * scale_log2;
    m[h] = m_new;
    l[h] *= corr[h];
  }
#pragma unroll
  for (int i = 0; i < NT; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float pv = exp2f(fmaf(s[i][e], scale_log2, shift[e >> 1]));
      s[i][e] = pv;
      l[e >> 1] += pv;
    }
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    o[i][0] *= corr[0]; o[i][1] *= corr[0];
    o[i][2] *= corr[1]; o[i][3] *= corr[1];
  }
}

// ---------------------------------------------------------------------------------------------
// Prefill / mixed steps.  One block per (tile of query rows, kv head); four warps of 16 rows.
// grid.x runs over an upper bound of the number of tiles; a block finds its request by walking
// query_start_loc.
// ---------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(FLASH_THREADS)
flash_prefill_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                     long long out_stride, const bf16* __restrict__ k_pages,
                     const bf16* __restrict__ v_pages, const int* __restrict__ block_table,
                     int table_stride, const int* __restrict__ query_start_loc,
                     const int* __restrict__ context_lens, int num_seqs, int page_shift,
                     int num_heads, int num_kv_heads, int window, float scale_log2) {
  pdl_wait();
  pdl_trigger<8>();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* k_s[2] = {reinterpret_cast<bf16*>(smem_raw), reinterpret_cast<bf16*>(smem_raw) + 2 * TILE_N * D};
  bf16* v_s[2] = {k_s[0] + TILE_N * D, k_s[1] + TILE_N * D};
  __shared__ int s_seq, s_tile;

  const int group = num_heads / num_kv_heads;
  const int tokens_per_tile = (FLASH_WARPS * 16) / group;
  if (threadIdx.x == 0) {
    // Blocks are handed out in launch order: the last tiles of a request (most keys under the
    // causal mask) are given the lowest block indices so that the longest blocks start first.
    int remaining = blockIdx.x, found = -1, tile = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int q_len = query_start_loc[s + 1] - query_start_loc[s];
      const int tiles = (q_len + tokens_per_tile - 1) / tokens_per_tile;
      if (remaining < tiles) { found = s; tile = tiles - 1 - remaining; break; }
      remaining -= tiles;
    }
    s_seq = found;
    s_tile = tile;
  }
  __syncthreads();
  const int seq = s_seq;
  if (seq < 0) return;
  const int kv_head = blockIdx.y;
  const int q_begin = query_start_loc[seq], q_len = query_start_loc[seq + 1] - q_begin;
  const int ctx = context_lens[seq];
  const int tok0 = s_tile * tokens_per_tile;                    // first query of the tile, in the request's portion
  const int tile_tokens = min(tokens_per_tile, q_len - tok0);
  const int pos0 = ctx - q_len + tok0;                          // its absolute position
  const int* table = block_table + (size_t)seq * table_stride;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  int pos[2], first[2];
  const bf16* q_rows[2];
  bf16* o_rows[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = warp * 16 + g + 8 * h;
    const int tok = row / group, head = kv_head * group + row % group;
    const bool valid = tok < tile_tokens;
    pos[h] = valid ? pos0 + tok : -1;
    first[h] = valid && window > 0 ? max(0, pos[h] - window + 1) : 0;
    q_rows[h] = valid ? q + (size_t)(q_begin + tok0 + tok) * q_stride + (size_t)head * D : nullptr;
    o_rows[h] = valid ? out + (size_t)(q_begin + tok0 + tok) * out_stride + (size_t)head * D : nullptr;
  }
  unsigned qf[D / 16][4];
  load_q_frags<D>(qf, q_rows[0], q_rows[1], t);
  // over the warp's rows that hold a query: the smallest position and the largest window start
  int warp_min_pos = min(pos[0] < 0 ? 0x7fffffff : pos[0], pos[1] < 0 ? 0x7fffffff : pos[1]);
  int warp_max_first = max(pos[0] < 0 ? 0 : first[0], pos[1] < 0 ? 0 : first[1]);
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    warp_min_pos = min(warp_min_pos, __shfl_xor_sync(0xffffffffu, warp_min_pos, offset));
    warp_max_first = max(warp_max_first, __shfl_xor_sync(0xffffffffu, warp_max_first, offset));
  }

  const int kv_first = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int kv_end = pos0 + tile_tokens;  // exclusive: the last query's own position + 1
  const int tile_begin = kv_first / TILE_N, tile_end = (kv_end + TILE_N - 1) / TILE_N;

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

  load_kv_tile<D>(k_s[0], v_s[0], k_pages, v_pages, table, tile_begin * TILE_N, kv_first, kv_end,
                  page_shift, num_kv_heads, kv_head);
  cp_async_commit();
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    const int stage = (tile - tile_begin) & 1;
    if (tile + 1 < tile_end)
      load_kv_tile<D>(k_s[stage ^ 1], v_s[stage ^ 1], k_pages, v_pages, table, (tile + 1) * TILE_N,
                      kv_first, kv_end, page_shift, num_kv_heads, kv_head);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    float s[8][4];
    qk_tile<D, 8>(s, qf, k_s[stage], 0, lane);
    // a tile needs the visibility tests only if it reaches past some row's position or starts
    // before some row's window
    if (tile * TILE_N + TILE_N - 1 > warp_min_pos || tile * TILE_N < warp_max_first)
      softmax_tile_raw<D, 8, true>(s, o, m, l, tile * TILE_N, t, pos, first, scale_log2);
    else
      softmax_tile_raw<D, 8, false>(s, o, m, l, tile * TILE_N, t, pos, first, scale_log2);
    pv_tile<D, 8>(o, s, v_s[stage], 0, lane);
    __syncthreads();
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float sum = l[h];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    if (o_rows[h]) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i)
        *reinterpret_cast<unsigned*>(o_rows[h] + i * 8 + 2 * t) = pack_bf16(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
  }
}

#define DECODE_CLUSTER_MAX 8  // the portable cluster size

__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of the same shared-memory location in block `rank` of this cluster.
__device__ __forceinline__ unsigned cluster_map(unsigned local, int rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}

// ---------------------------------------------------------------------------------------------
// The end of a decode block, shared by the two decode kernels: the block's warps (each with its
// own running softmax over its keys) are joined through shared memory; then the block writes the
// output row (one split), its partial result to scratch (splits joined by a second kernel), or,
// as one block of a cluster, leaves its partial in shared memory and joins its share of the
// cluster's results over distributed shared memory.  Every thread of the block calls it;
// `active` is false for threads that hold no result (a producer warp).
// ---------------------------------------------------------------------------------------------
// SLOTS: how many partial results meet in the block's join area: one per consumer warp, and with
// FLASH_WARPS + 1 one more that the caller has filled in before the call (rows of [16][D] floats
// at decode_join_o(smem_raw) + FLASH_WARPS * 16 * D, their (max, sum) at decode_join_ml<D, SLOTS>
// (smem_raw) + FLASH_WARPS * 16 * 2; a max of -inf gives the slot no weight and its rows are not read).
template <int D> __device__ __forceinline__ float* decode_join_o(unsigned char* smem_raw) {
  return reinterpret_cast<float*>(smem_raw);
}
template <int D, int SLOTS> __device__ __forceinline__ float* decode_join_ml(unsigned char* smem_raw) {
  return reinterpret_cast<float*>(smem_raw) + SLOTS * 16 * D;
}

template <int D, bool CLUSTER, int SLOTS = FLASH_WARPS>
__device__ __forceinline__ void decode_finish(float (&o)[D / 8][4], float (&m)[2], float (&l)[2], unsigned char* smem_raw,
                                              bool active, int warp, int lane, int group, int kv_head, int token,
                                              int split, int num_splits, int num_heads, bf16* __restrict__ out,
                                              long long out_stride, float* __restrict__ partial_o,
                                              float* __restrict__ partial_ml, long long slot0 = -1,
                                              long long slot_stride = 0) {
  const int g = lane >> 2, t = lane & 3;
  // where this block's partial result of head h goes in scratch: slot0 + h * slot_stride; by
  // default the layout [tokens, heads, splits]
  if (slot0 < 0) {
    slot0 = (long long)token * num_heads * num_splits + split;
    slot_stride = num_splits;
  }
  // each warp writes (m, l) per row and its O tile; then all read them
  float* join_o = decode_join_o<D>(smem_raw);                    // [SLOTS][16][D]
  float* join_ml = decode_join_ml<D, SLOTS>(smem_raw);           // [SLOTS][16][2]
#pragma unroll
  for (int h = 0; h < 2 && active; ++h) {
    float sum = l[h];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l[h] = sum;
    const int row = g + 8 * h;
    if (t == 0) {
      join_ml[(warp * 16 + row) * 2] = m[h];
      join_ml[(warp * 16 + row) * 2 + 1] = sum;
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      join_o[(warp * 16 + row) * D + i * 8 + 2 * t] = o[i][2 * h];
      join_o[(warp * 16 + row) * D + i * 8 + 2 * t + 1] = o[i][2 * h + 1];
    }
  }
  __syncthreads();
  // thread -> (row, dims): 128 threads cover 16 rows x D dims, D/8 dims each
  for (int idx = active ? (int)threadIdx.x : group * (D / 4); idx < group * (D / 4); idx += FLASH_THREADS) {
    const int row = idx / (D / 4), d0 = (idx % (D / 4)) * 4;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < SLOTS; ++w) m_all = fmaxf(m_all, join_ml[(w * 16 + row) * 2]);
    float l_all = 0.0f, acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int w = 0; w < SLOTS; ++w) {
      const float mw = join_ml[(w * 16 + row) * 2];
      if (mw == -INFINITY) continue;  // a slot without keys: no weight, and its rows may hold anything
      const float wgt = exp2f(mw - m_all);
      l_all += join_ml[(w * 16 + row) * 2 + 1] * wgt;
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[e] += join_o[(w * 16 + row) * D + d0 + e] * wgt;
    }
    const int head = kv_head * group + row;
    if (CLUSTER) {
      float* mine_o = join_ml + SLOTS * 16 * 2;  // [16][D] then [16][2], behind the warps' join area
      float* mine_ml = mine_o + 16 * D;
      *reinterpret_cast<float4*>(mine_o + row * D + d0) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      if (d0 == 0) {
        mine_ml[row * 2] = m_all;
        mine_ml[row * 2 + 1] = l_all;
      }
    } else if (num_splits == 1) {
      const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
      bf16* dst = out + (size_t)token * out_stride + (size_t)head * D + d0;
      *reinterpret_cast<unsigned*>(dst) = pack_bf16(acc[0] * inv, acc[1] * inv);
      *reinterpret_cast<unsigned*>(dst + 2) = pack_bf16(acc[2] * inv, acc[3] * inv);
    } else {
      const size_t slot = (size_t)(slot0 + (long long)head * slot_stride);
      float* dst = partial_o + slot * D + d0;
      *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      if (d0 == 0) {
        partial_ml[slot * 2] = m_all;
        partial_ml[slot * 2 + 1] = l_all;
      }
    }
  }
  if (CLUSTER) {
    // every block of the cluster reaches this point (a padding token sends all of them away
    // together at the top); the barrier makes the partials visible across the cluster
    cluster_barrier();
    const unsigned mine_o = smem_u32(join_ml + SLOTS * 16 * 2);
    const unsigned mine_ml = mine_o + 16 * D * (unsigned)sizeof(float);
    for (int idx = active ? split * FLASH_THREADS + (int)threadIdx.x : group * (D / 4); idx < group * (D / 4); idx += num_splits * FLASH_THREADS) {
      const int row = idx / (D / 4), d0 = (idx % (D / 4)) * 4;
      float ms[DECODE_CLUSTER_MAX], ls[DECODE_CLUSTER_MAX];
      float m_all = -INFINITY;
#pragma unroll
      for (int r = 0; r < DECODE_CLUSTER_MAX; ++r) {
        ms[r] = -INFINITY;
        ls[r] = 0.0f;
        if (r < num_splits) {
          const unsigned remote = cluster_map(mine_ml + (unsigned)(row * 2) * 4u, r);
          asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];" : "=f"(ms[r]), "=f"(ls[r]) : "r"(remote));
          m_all = fmaxf(m_all, ms[r]);
        }
      }
      float l_all = 0.0f, acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int r = 0; r < DECODE_CLUSTER_MAX; ++r) {
        if (r < num_splits) {
          const float wgt = ms[r] == -INFINITY ? 0.0f : exp2f(ms[r] - m_all);
          l_all += ls[r] * wgt;
          float4 part;
          const unsigned remote = cluster_map(mine_o + (unsigned)(row * D + d0) * 4u, r);
          asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];"
                       : "=f"(part.x), "=f"(part.y), "=f"(part.z), "=f"(part.w) : "r"(remote));
          acc[0] += part.x * wgt; acc[1] += part.y * wgt; acc[2] += part.z * wgt; acc[3] += part.w * wgt;
        }
      }
      const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
      bf16* dst = out + (size_t)token * out_stride + (size_t)(kv_head * group + row) * D + d0;
      *reinterpret_cast<unsigned*>(dst) = pack_bf16(acc[0] * inv, acc[1] * inv);
      *reinterpret_cast<unsigned*>(dst + 2) = pack_bf16(acc[2] * inv, acc[3] * inv);
    }
    cluster_barrier();  // no block leaves while another may still read its shared memory
  }
}

// ---------------------------------------------------------------------------------------------
// Decode steps: one query token per request.  One block per (split, kv head, request); the
// group's heads are the rows (at most 16).  The block stages 64-key tiles together; warp w
// scores keys 16w .. 16w+15 of each tile and keeps its own running softmax; the four warps are
// joined through shared memory.  With more than one split the block writes its unnormalised
// result and (max, sum) to scratch, else the output row.
//   partial_o:  [tokens, heads, splits, D] fp32      partial_ml: [tokens, heads, splits, 2] fp32
// CLUSTER: the splits of one (kv head, request) are the blocks of one thread-block cluster (at
// most DECODE_CLUSTER_MAX of them); each leaves its partial result in its own shared memory and,
// after a cluster barrier, the blocks share out the (head, dims) items and join them by reading
// every block's partials over distributed shared memory: no scratch, no second kernel.
// ---------------------------------------------------------------------------------------------
template <int D, bool CLUSTER>
__global__ void __launch_bounds__(FLASH_THREADS)
flash_decode_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                    long long out_stride, const bf16* __restrict__ k_pages,
                    const bf16* __restrict__ v_pages, const int* __restrict__ block_table,
                    int table_stride, const int* __restrict__ seq_of_token,
                    const int* __restrict__ positions, int page_shift, int num_heads,
                    int num_kv_heads, int window, float scale_log2, int num_splits,
                    float* __restrict__ partial_o, float* __restrict__ partial_ml, int* __restrict__ status) {
  pdl_wait();
  pdl_trigger<8>();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  bf16* const ring = reinterpret_cast<bf16*>(smem_raw);  // DECODE_STAGES x (K tile, V tile)

  const int split = blockIdx.x, kv_head = blockIdx.y, token = blockIdx.z;
  const int seq = seq_of_token[token];
  if (seq < 0) return;
  const int group = num_heads / num_kv_heads;
  const int pos = positions[token];
  const int kv_first = window > 0 ? max(0, pos - window + 1) : 0;
  const int num_keys = pos + 1 - kv_first;
  int chunk = (num_keys + num_splits - 1) / num_splits;
  chunk = (chunk + TILE_N - 1) / TILE_N * TILE_N;
  const int begin = kv_first + split * chunk;
  const int end = min(pos + 1, begin + chunk);
  const int* table = block_table + (size_t)seq * table_stride;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

  if (begin < end) {
    int rpos[2], rfirst[2];
    const bf16* q_rows[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = g + 8 * h;
      const bool valid = row < group;
      rpos[h] = valid ? pos : -1;
      rfirst[h] = kv_first;
      q_rows[h] = valid ? q + (size_t)token * q_stride + (size_t)(kv_head * group + row) * D : nullptr;
    }
    // Every warp streams its own 16-key tiles (tiles warp, warp + 4, ... of the block's range):
    // no block-wide barrier in the loop.  Keys never touch shared memory: the thread (g, t) loads
    // 16 bytes (dims 32c + 8t .. + 7) of key g of each 8-key group straight into the mma B
    // fragment, with the query fragment read by the same rule (a one-to-one assignment of dims to
    // k-slots leaves a dot product unchanged); two tiles of keys are in flight in registers.
    // Values need the transposed load, so they go through a private shared-memory ring of
    // DECODE_STAGES tiles.  Registers and ring together keep ~190 KB per SM in flight, which is
    // what it takes to keep HBM busy (measured: 128 KB in flight gives 4.3 TB/s, this 5.2).
    constexpr int WARP_TILE = 16;
    constexpr int CH = D / 8;    // 16-byte chunks per row
    constexpr int CHK = D / 32;  // 32-dim chunks per row
    const int num_tiles = (end - begin + WARP_TILE - 1) / WARP_TILE;
    const int my_tiles = num_tiles > warp ? (num_tiles - warp + FLASH_WARPS - 1) / FLASH_WARPS : 0;
    const int page_mask = (1 << page_shift) - 1;

    uint4 q_lo[CHK], q_hi[CHK];
#pragma unroll
    for (int c = 0; c < CHK; ++c) {
      q_lo[c] = q_rows[0] ? *reinterpret_cast<const uint4*>(q_rows[0] + 32 * c + 8 * t) : make_uint4(0u, 0u, 0u, 0u);
      q_hi[c] = q_rows[1] ? *reinterpret_cast<const uint4*>(q_rows[1] + 32 * c + 8 * t) : make_uint4(0u, 0u, 0u, 0u);
    }

    // A key in range whose page is missing from the table (given back too early: a fault of whoever
    // made the table) is masked out of the softmax and raises bit 4 of *status.  found[j] has bit
    // 4 * r set when key 8 * j + r of the tile has its page.
    auto load_keys = [&](uint4 (&kr)[2][CHK], unsigned (&found)[2], int i) {  // the i-th tile of this warp, into registers
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int key = begin + (warp + i * FLASH_WARPS) * WARP_TILE + 8 * j + g;
        bool ok = i < my_tiles && key < end;
        const int page = ok ? table[key >> page_shift] : -1;
        const bool missing = ok && page < 0;
        found[j] = __ballot_sync(0xffffffffu, !missing);
        if (missing && t == 0 && status) atomicOr(status, 4);
        ok = ok && page >= 0;
        const bf16* row = k_pages + ((((size_t)(ok ? page : 0) << page_shift) + (key & page_mask)) * num_kv_heads + kv_head) * D + 8 * t;
#pragma unroll
        for (int c = 0; c < CHK; ++c) {
          kr[j][c] = make_uint4(0u, 0u, 0u, 0u);
          if (ok)
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(kr[j][c].x), "=r"(kr[j][c].y), "=r"(kr[j][c].z), "=r"(kr[j][c].w)
                         : "l"(row + 32 * c));
        }
      }
    };
    bf16* const my_ring = ring + warp * DECODE_STAGES * WARP_TILE * D;
    const int load_row = lane >> 1, load_half = lane & 1;
    auto load_values = [&](int i) {  // the i-th tile of this warp, into the ring
      const unsigned v_base = smem_u32(my_ring + (i % DECODE_STAGES) * WARP_TILE * D);
      const int key = begin + (warp + i * FLASH_WARPS) * WARP_TILE + load_row;
      bool ok = key < end;
      const int page = ok ? table[key >> page_shift] : -1;
      ok = ok && page >= 0;
      const size_t off = ok ? ((((size_t)page << page_shift) + (key & page_mask)) * num_kv_heads + kv_head) * D : 0;
#pragma unroll
      for (int j = 0; j < CH / 2; ++j) {
        const int c = 2 * j + load_half;
        cp_async16(v_base + tile_offset<D>(load_row, c), v_pages + off + c * 8, ok ? 16 : 0);
      }
    };

    uint4 k0[2][CHK], k1[2][CHK], k2[2][CHK];
    unsigned f0[2], f1[2], f2[2];
    load_keys(k0, f0, 0);
    load_keys(k1, f1, 1);
#pragma unroll
    for (int s = 0; s < DECODE_STAGES - 1; ++s) {
      if (s < my_tiles) load_values(s);
      cp_async_commit();
    }
    for (int i = 0; i < my_tiles; ++i) {
      load_keys(k2, f2, i + 2);
      if (i + DECODE_STAGES - 1 < my_tiles) load_values(i + DECODE_STAGES - 1);
      cp_async_commit();
      const int key0 = begin + (warp + i * FLASH_WARPS) * WARP_TILE;
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
#pragma unroll
        for (int c = 0; c < CHK; ++c) {
          const unsigned a_first[4] = {q_lo[c].x, q_hi[c].x, q_lo[c].y, q_hi[c].y};
          const unsigned a_second[4] = {q_lo[c].z, q_hi[c].z, q_lo[c].w, q_hi[c].w};
          mma16816(s[j], a_first, k0[j][c].x, k0[j][c].y);
          mma16816(s[j], a_second, k0[j][c].z, k0[j][c].w);
        }
        if (f0[j] != 0xffffffffu) {  // element e of this thread is key 8 * j + 2 * t + (e & 1)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (!((f0[j] >> (4 * (2 * t + (e & 1)))) & 1u)) s[j][e] = -INFINITY;
        }
      }
      int limit[2] = {min(rpos[0], end - 1), min(rpos[1], end - 1)};
      softmax_tile<D, 2>(s, o, m, l, key0, t, limit, rfirst, scale_log2);
      cp_async_wait<DECODE_STAGES - 1>();
      __syncwarp();
      pv_tile<D, 2>(o, s, my_ring + (i % DECODE_STAGES) * WARP_TILE * D, 0, lane);
      __syncwarp();  // the tile is free before a later iteration's copies land in it
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int c = 0; c < CHK; ++c) {
          k0[j][c] = k1[j][c];
          k1[j][c] = k2[j][c];
        }
      f0[0] = f1[0]; f0[1] = f1[1];
      f1[0] = f2[0]; f1[1] = f2[1];
    }
    cp_async_wait<0>();
    __syncthreads();  // every warp is done with its ring before the join reuses the memory
  }

  decode_finish<D, CLUSTER>(o, m, l, smem_raw, true, warp, lane, group, kv_head, token, split, num_splits, num_heads, out,
                            out_stride, partial_o, partial_ml);
}

// ---------------------------------------------------------------------------------------------
// Decode steps, head size 128, keys and values fetched by TMA.  The kernel above asks for its
// keys and values 16 bytes per lane at a time: thousands of requests per block, which the load
// queues of an SM hand out at their own pace (issuing a block's first tiles takes 4 of its 23 us).
// Here one lane per page issues bulk tensor copies of whole pages (one box per page and 64-dim
// half, 128-byte swizzle) into a ring of three stages of 64 keys, 32 KB each, guarded by
// mbarriers; four warps take 16 keys of every stage each (ldmatrix from the swizzled tiles, the
// same mma.sync arithmetic as the tiled kernel) and keep their own running softmax; the end of
// the block is decode_finish() as above.  A block covers whole 64-key tiles of the request's keys
// (aligned to 64 from key 0, so that a box never straddles a page); keys before the window or
// after the position are masked.  Every mbarrier wait is bounded: one that runs out raises bit 64
// of *status and the block goes to its end with what it has.
// ---------------------------------------------------------------------------------------------
#define DTMA_KEYS 64
#define DTMA_STAGES 3
#define DTMA_HALF 8192          // [64 keys x 64 dims] bf16
#define DTMA_THREADS (FLASH_THREADS + 32)
#define DTMA_SMEM(D) (DTMA_STAGES * 2 * ((D) / 64) * DTMA_HALF + 1024)
#define DTMA_WAIT_LIMIT (1 << 24)

__device__ __forceinline__ void dtma_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void dtma_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void dtma_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool dtma_try_wait(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool dtma_wait(unsigned bar, unsigned parity, volatile int* failed) {
  for (int i = 0; i < DTMA_WAIT_LIMIT; ++i) {
    if (dtma_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023 && *failed) return false;
  }
  return false;
}
__device__ __forceinline__ void dtma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// byte offset of 16-byte chunk c (of 16) of key row r in a stage's keys or values: two half tiles
// of [64 rows x 128 bytes], chunks swizzled by the row as TMA's 128-byte mode leaves them
__device__ __forceinline__ unsigned dtma_offset(int r, int c) {
  return (unsigned)((c >> 3) * DTMA_HALF + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}

// A work list for decode steps whose requests differ much in length: item i is part
// item_part[i] of token item_token[i] (-1: unused); token t is cut into parts_of[t] parts, whose
// items lie one after the other from first_item[t].  All null: no list, every token is cut into
// the same number of parts by the grid.
struct DecodeItems {
  const int* item_token;
  const int* item_part;
  const int* parts_of;
  const int* first_item;
};

// What the kernel needs to do the step before attention itself (FUSED): the raw q/k/v product of
// the step's tokens, the bias, the rotation's constants, and the pages to append to.  The block
// of a (request, kv head) adds the bias to its query heads and rotates them (fp32, rounded to
// bfloat16 once, the arithmetic of rope_cache_write_kernel in layer_ops.cu bit for bit); the
// block whose keys end at the token's own position does the same for the token's key, appends
// key and value to the cache, and brings them into the softmax as one more partial result (a
// score, a sum of 1, the value as the output), while the keys from the cache stop one position
// earlier.  Nothing the kernel before wrote is needed for the keys and values of earlier
// positions, so their copies are under way before the kernel waits for the projections.
struct DecodeFusion {
  const bf16* qkv;        // [tokens, qkv_stride]: query heads, then key heads, then value heads, 128 wide each
  long long qkv_stride;
  const float* bias;      // [(num_heads + 2 * num_kv_heads) * 128] or null
  const float* inv_freq;  // [rotary_dim / 2] or null when rotary_dim == 0
  int rotary_dim;         // even, at most 128; pairs (i, i + rotary_dim / 2) are rotated
  float factor;           // positions are divided by it
  bf16* k_pages;          // [pages, page_size, kv_heads, 128], appended to when write_kv
  bf16* v_pages;
  int write_kv;
};

#define DTMA_Q_STRIDE 136  // bf16 elements per row of the rotated queries in shared memory (272 bytes: no bank conflicts)

__device__ __forceinline__ void dtma_rotate(float x1, float x2, float c, float s, float& o1, float& o2) {
  o1 = __fmaf_rn(x1, c, -__fmul_rn(x2, s));  // the roundings of rope_rotate() in layer_ops.cu
  o2 = __fmaf_rn(x2, c, __fmul_rn(x1, s));
}

template <int D, bool CLUSTER, bool FUSED>
__global__ void __launch_bounds__(DTMA_THREADS, 2)
flash_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                        long long out_stride, const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                        int page_shift, int box_rows, int total_rows, int num_heads, int num_kv_heads,
                        int window, float scale_log2, int num_splits, float* __restrict__ partial_o,
                        float* __restrict__ partial_ml, int* __restrict__ status, const DecodeFusion fusion,
                        const DecodeItems items) {
  static_assert(D == 64 || D == 128, "head size 64 or 128");
  static_assert(!FUSED || D == 128, "the kernel encodes and appends itself for head size 128 only");
  constexpr int HALVES = D / 64;                           // 64-dim halves of a key or value row
  constexpr int STAGE_BYTES = 2 * HALVES * DTMA_HALF;      // keys (their halves), then values (theirs)
  constexpr int SLOTS = FUSED ? FLASH_WARPS + 1 : FLASH_WARPS;
  if (!FUSED) pdl_wait();  // no early trigger: with it the decode step was 0.2 ms slower (3.42 against 3.21 ms)
  extern __shared__ unsigned char dtma_raw[];
  __shared__ __align__(8) unsigned long long bars[2 * DTMA_STAGES];
  __shared__ int failed;
  __shared__ unsigned gone_s[DTMA_STAGES];  // per stage: bit b set when box b lies on a page that is missing from the table
  __shared__ __align__(16) bf16 q_s[FUSED ? 16 * DTMA_Q_STRIDE : 8];  // rotated queries, rows = heads of the group
  __shared__ __align__(16) bf16 kv_s[FUSED ? 2 * D : 8];               // the token's own key (rotated), then value
  __shared__ float cs_s[FUSED ? D : 2];                                 // cos, then sin, of the token's angles

  // Which part of which token this block works on: by its place in the grid (every token cut
  // into num_splits parts), or, with a work list, by item blockIdx.x of the list, whose tokens are
  // cut into as many parts as their own length asks for (items.parts_of) and leave their partial
  // results at [items.first_item[token] + part][head] of the scratch.
  int split = blockIdx.x, token = blockIdx.z;
  const int kv_head = blockIdx.y;
  long long slot0 = -1;
  if (items.item_token != nullptr) {
    token = items.item_token[blockIdx.x];
    if (token < 0) {  // an unused item
      if (FUSED) pdl_wait();
      return;
    }
    split = items.item_part[blockIdx.x];
    num_splits = items.parts_of[token];
    slot0 = (long long)(items.first_item[token] + split) * num_heads;
  }
  const int seq = seq_of_token[token];
  if (seq < 0) {  // the same for every block of a cluster: nothing has been set up
    if (FUSED) pdl_wait();
    return;
  }
  const int group = num_heads / num_kv_heads;
  const int pos = positions[token];
  const int last_cached = FUSED ? pos - 1 : pos;  // the last key that comes from the cache
  const int kv_first = window > 0 ? max(0, pos - window + 1) : 0;
  const int tile_begin = kv_first / DTMA_KEYS, tile_end = pos / DTMA_KEYS + 1;
  const int per_split = (tile_end - tile_begin + num_splits - 1) / num_splits;
  const int my_begin = tile_begin + split * per_split;
  const int num_tiles = max(0, min(tile_end, my_begin + per_split) - my_begin);
  // the part whose keys end at the token's own position: it appends the token's key and value
  const bool owner = FUSED && split == (tile_end - 1 - tile_begin) / per_split;
  const int* table = block_table + (size_t)seq * table_stride;
  if (!CLUSTER && num_splits > 1 && num_tiles == 0) {
    // a part without keys (a short request in a batch that is cut for a long one): no weight in the
    // join, and nothing else to do (the same for every thread; nothing has been set up)
    if (FUSED) pdl_wait();
    if ((int)threadIdx.x < group) {
      const int head = kv_head * group + threadIdx.x;
      const size_t slot = slot0 >= 0 ? (size_t)(slot0 + head) : ((size_t)token * num_heads + head) * num_splits + split;
      partial_ml[slot * 2] = -INFINITY;
      partial_ml[slot * 2 + 1] = 0.0f;
    }
    return;
  }

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const unsigned ring = (smem_u32(dtma_raw) + 1023u) & ~1023u;
  unsigned char* const ring_ptr = dtma_raw + (ring - smem_u32(dtma_raw));
  const unsigned full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[DTMA_STAGES]);
  if (threadIdx.x == 0) {
    failed = 0;
    for (int st = 0; st < DTMA_STAGES; ++st) {
      dtma_mbar_init(full0 + 8 * st, 1);
      dtma_mbar_init(empty0 + 8 * st, FLASH_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[i][e] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

  // ---- producer (warp FLASH_WARPS): one lane per box (a page, or 64 keys of a larger page) ----------
  const int page_size = 1 << page_shift;
  const int boxes = DTMA_KEYS / box_rows;
  bool producer_ok = true;
  auto issue_tiles = [&](int from, int to) {
    for (int it = from; it < to && producer_ok; ++it) {
      const int st = it % DTMA_STAGES;
      if (it >= DTMA_STAGES && !__all_sync(0xffffffffu, dtma_wait(empty0 + 8 * st, ((it / DTMA_STAGES) - 1) & 1, &failed))) {
        if (lane == 0) {
          failed = 1;
          if (status) atomicOr(status, 64);
        }
        producer_ok = false;
        break;
      }
      const int key = (my_begin + it) * DTMA_KEYS + lane * box_rows;
      int row = total_rows;  // out of range: the box is filled with zeros
      bool gone = false;
      if (lane < boxes && key <= last_cached && key + box_rows > kv_first) {
        const int page = table[key >> page_shift];
        if (page >= 0) row = page * page_size + (key & (page_size - 1));
        else gone = true;  // a page in reach of this block is missing: its keys get no weight
      }
      const unsigned gone_boxes = __ballot_sync(0xffffffffu, gone);
      if (lane == 0) {
        if (gone_boxes && status) atomicOr(status, 4);
        gone_s[st] = gone_boxes;  // before the arrival below, which releases it to the consumers
        dtma_expect_tx(full0 + 8 * st, STAGE_BYTES);
      }
      __syncwarp();
      if (lane < boxes) {
        const unsigned dst = ring + st * STAGE_BYTES + lane * box_rows * 128;
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
          dtma_load_2d(dst + h * DTMA_HALF, &map_k, kv_head * D + h * 64, row, full0 + 8 * st);
          dtma_load_2d(dst + (HALVES + h) * DTMA_HALF, &map_v, kv_head * D + h * 64, row, full0 + 8 * st);
        }
      }
    }
  };

  if (FUSED) {
    // Before the wait: the first stages of keys and values (positions before the token's own: no
    // kernel of this step has written them) and the token's angles.
    const int ahead = min(num_tiles, DTMA_STAGES);
    if (warp == FLASH_WARPS) issue_tiles(0, ahead);
    const int half = fusion.rotary_dim / 2;
    if ((int)threadIdx.x < half) {
      float sn, cn;
      sincosf(((float)pos / fusion.factor) * fusion.inv_freq[threadIdx.x], &sn, &cn);
      cs_s[threadIdx.x] = cn;
      cs_s[64 + threadIdx.x] = sn;
    }
    pdl_wait();
    __syncthreads();
    // rotated queries of the group's heads, and (owner) the token's key and value: rows
    // 0 .. group - 1 are queries, row `group` the key, row `group + 1` the value
    const bf16* x_row = fusion.qkv + (size_t)token * fusion.qkv_stride;
    const int rows = owner ? group + 2 : group;
    // Item (r, i), i < 64: elements i and i + 64 of row r (at most 18 rows: 16 heads, key, value).
    // All loads of a thread are issued before the first result is needed: one trip to memory.
    constexpr int ITEMS = (18 * 64 + DTMA_THREADS - 1) / DTMA_THREADS;
    float xa[ITEMS], xb[ITEMS];
#pragma unroll
    for (int u = 0; u < ITEMS; ++u) {
      const int idx = threadIdx.x + u * DTMA_THREADS;
      xa[u] = xb[u] = 0.0f;
      if (idx < rows * 64) {
        const int r = idx >> 6, i = idx & 63;
        const int head = r < group ? kv_head * group + r : (r == group ? num_heads + kv_head : num_heads + num_kv_heads + kv_head);
        const bf16* x = x_row + (size_t)head * D;
        xa[u] = __bfloat162float(x[i]);
        xb[u] = __bfloat162float(x[i + 64]);
        if (fusion.bias) {
          xa[u] += fusion.bias[(size_t)head * D + i];
          xb[u] += fusion.bias[(size_t)head * D + i + 64];
        }
      }
    }
    // Elements e < half are rotated with e + half; elements from 2 * half on pass through.  With
    // i < 64 <= D / 2 the pair of item i is (i, i + half) only when half == 64; for a narrower
    // rotation the partner of element i lies in another item, so it is fetched again from the row.
#pragma unroll
    for (int u = 0; u < ITEMS; ++u) {
      const int idx = threadIdx.x + u * DTMA_THREADS;
      if (idx < rows * 64) {
        const int r = idx >> 6, i = idx & 63;
        const bool is_value = r == group + 1;
        bf16* dst = r < group ? q_s + r * DTMA_Q_STRIDE : kv_s + (r - group) * D;
        if (is_value || half == 0) {
          dst[i] = __float2bfloat16_rn(xa[u]);
          dst[i + 64] = __float2bfloat16_rn(xb[u]);
        } else if (half == 64) {
          float o1, o2;
          dtma_rotate(xa[u], xb[u], cs_s[i], cs_s[64 + i], o1, o2);
          dst[i] = __float2bfloat16_rn(o1);
          dst[i + 64] = __float2bfloat16_rn(o2);
        } else {
          // a rotation narrower than the head: both of this item's elements on their own
          const int head = r < group ? kv_head * group + r : num_heads + kv_head;
          const bf16* x = x_row + (size_t)head * D;
          const float* b = fusion.bias ? fusion.bias + (size_t)head * D : nullptr;
#pragma unroll
          for (int which = 0; which < 2; ++which) {
            const int e = i + 64 * which;
            const float own = which ? xb[u] : xa[u];
            float result = own;
            if (e < 2 * half) {
              const int partner = e < half ? e + half : e - half;
              float other = __bfloat162float(x[partner]);
              if (b) other += b[partner];
              float o1, o2;
              if (e < half) { dtma_rotate(own, other, cs_s[e], cs_s[64 + e], o1, o2); result = o1; }
              else { dtma_rotate(other, own, cs_s[partner], cs_s[64 + partner], o1, o2); result = o2; }
            }
            dst[e] = __float2bfloat16_rn(result);
          }
        }
      }
    }
    for (int idx = group * DTMA_Q_STRIDE + threadIdx.x; idx < 16 * DTMA_Q_STRIDE; idx += DTMA_THREADS)
      q_s[idx] = __float2bfloat16_rn(0.0f);  // rows without a query
    __syncthreads();
    if (owner && fusion.write_kv && threadIdx.x < 32) {
      // append: 16 threads copy the key, 16 the value, 16 bytes each
      const int page = table[pos >> page_shift];
      if (page < 0) {
        if (threadIdx.x == 0 && status) atomicOr(status, 2);
      } else {
        const int which = threadIdx.x >> 4, chunk = threadIdx.x & 15;
        bf16* pages = which ? fusion.v_pages : fusion.k_pages;
        bf16* dst = pages + (((size_t)page * page_size + (pos & (page_size - 1))) * num_kv_heads + kv_head) * D;
        *reinterpret_cast<uint4*>(dst + chunk * 8) = *reinterpret_cast<const uint4*>(kv_s + which * D + chunk * 8);
      }
    }
    if (warp == FLASH_WARPS) issue_tiles(ahead, num_tiles);
  } else if (warp == FLASH_WARPS) {
    issue_tiles(0, num_tiles);
  }

  if (warp < FLASH_WARPS && num_tiles > 0) {
    // ---- consumers: warp w takes keys 16w .. 16w + 15 of every stage ------------------------------
    int rpos[2], rfirst[2];
    const bf16* q_rows[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = g + 8 * h;
      const bool valid = row < group;
      rpos[h] = valid ? last_cached : -1;
      rfirst[h] = kv_first;
      if (FUSED) q_rows[h] = q_s + row * DTMA_Q_STRIDE;  // rows without a query are zero
      else q_rows[h] = valid ? q + (size_t)token * q_stride + (size_t)(kv_head * group + row) * D : nullptr;
    }
    unsigned qf[D / 16][4];
    load_q_frags<D>(qf, q_rows[0], q_rows[1], t);
    const int mi = lane >> 3, lr = lane & 7;
    const int key_row_k = 16 * warp + (mi >> 1) * 8 + lr, key_row_v = 16 * warp + (mi & 1) * 8 + lr;
    for (int it = 0; it < num_tiles; ++it) {
      const int st = it % DTMA_STAGES;
      if (!__all_sync(0xffffffffu, dtma_wait(full0 + 8 * st, (it / DTMA_STAGES) & 1, &failed))) {
        if (lane == 0) {
          failed = 1;
          if (status) atomicOr(status, 64);
        }
        break;
      }
      const unsigned keys = ring + st * STAGE_BYTES, values = keys + HALVES * DTMA_HALF;
      float sc[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[i][e] = 0.0f;
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        unsigned b[4];
        ldmatrix_x4(b, keys + dtma_offset(key_row_k, kk * 2 + (mi & 1)));
        mma16816(sc[0], qf[kk], b[0], b[1]);
        mma16816(sc[1], qf[kk], b[2], b[3]);
      }
      const int key0 = (my_begin + it) * DTMA_KEYS + 16 * warp;
      const unsigned gone_boxes = gone_s[st];
      if (gone_boxes) {  // element e of sc[i] is key 16 * warp + 8 * i + 2 * t + (e & 1) of the stage
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if ((gone_boxes >> ((16 * warp + 8 * i + 2 * t + (e & 1)) / box_rows)) & 1u) sc[i][e] = -INFINITY;
      }
      softmax_tile<D, 2>(sc, o, m, l, key0, t, rpos, rfirst, scale_log2);
      unsigned a[4];
      a[0] = pack_bf16(sc[0][0], sc[0][1]);
      a[1] = pack_bf16(sc[0][2], sc[0][3]);
      a[2] = pack_bf16(sc[1][0], sc[1][1]);
      a[3] = pack_bf16(sc[1][2], sc[1][3]);
#pragma unroll
      for (int np = 0; np < D / 16; ++np) {
        unsigned b[4];
        ldmatrix_x4_trans(b, values + dtma_offset(key_row_v, np * 2 + (mi >> 1)));
        mma16816(o[2 * np], a, b[0], b[1]);
        mma16816(o[2 * np + 1], a, b[2], b[3]);
      }
      __syncwarp();
      if (lane == 0) dtma_arrive(empty0 + 8 * st);  // this warp has read its rows of the stage
    }
  }
  __syncthreads();  // every warp is done with the ring before the join reuses the memory
  if (failed && threadIdx.x == 0) {
    // copies that were issued may still be landing: give them a bounded while
    for (int st = 0; st < DTMA_STAGES; ++st)
      for (int i = 0; i < 4096 && !dtma_try_wait(full0 + 8 * st, 0) && !dtma_try_wait(full0 + 8 * st, 1); ++i) {}
  }
  if (FUSED && warp == FLASH_WARPS) {
    // the token's own key and value as one more partial result: score, a sum of 1, the value
    float* extra_o = decode_join_o<D>(ring_ptr) + FLASH_WARPS * 16 * D;
    float* extra_ml = decode_join_ml<D, SLOTS>(ring_ptr) + FLASH_WARPS * 16 * 2;
    float kd[4], vd[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      kd[e] = __bfloat162float(kv_s[4 * lane + e]);
      vd[e] = __bfloat162float(kv_s[D + 4 * lane + e]);
    }
    for (int row = 0; row < 16; ++row) {
      float score = -INFINITY;
      if (owner && row < group) {
        float dot = 0.0f;
#pragma unroll
        for (int e = 0; e < 4; ++e) dot += __bfloat162float(q_s[row * DTMA_Q_STRIDE + 4 * lane + e]) * kd[e];
        score = warp_sum(dot) * scale_log2;
        *reinterpret_cast<float4*>(extra_o + row * D + 4 * lane) = make_float4(vd[0], vd[1], vd[2], vd[3]);
      }
      if (lane == 0) {
        extra_ml[row * 2] = score;
        extra_ml[row * 2 + 1] = score == -INFINITY ? 0.0f : 1.0f;
      }
    }
  }
  decode_finish<D, CLUSTER, SLOTS>(o, m, l, ring_ptr, warp < FLASH_WARPS, warp, lane, group, kv_head, token, split,
                                   num_splits, num_heads, out, out_stride, partial_o, partial_ml, slot0, 1);
}

// Join the splits of a decode step: one block per (token, head), one thread per dim.
template <int D>
__global__ void __launch_bounds__(D)
flash_decode_join_kernel(bf16* __restrict__ out, long long out_stride,
                         const int* __restrict__ seq_of_token, int num_heads, int num_splits,
                         const float* __restrict__ partial_o, const float* __restrict__ partial_ml,
                         const int* __restrict__ parts_of, const int* __restrict__ first_item) {
  pdl_wait();
  pdl_trigger<8>();
  const int head = blockIdx.x, token = blockIdx.y;
  if (seq_of_token[token] < 0) return;
  // part s of this (token, head) is at slot0 + s * stride: [tokens, heads, splits], or with a work
  // list [items, heads] with the token's items one after the other
  size_t slot0 = ((size_t)token * num_heads + head) * num_splits, stride = 1;
  if (parts_of != nullptr) {
    num_splits = parts_of[token];
    if (num_splits == 1) return;  // the one part wrote the output row itself
    slot0 = (size_t)first_item[token] * num_heads + head;
    stride = num_heads;
  }
  float m_all = -INFINITY;
  for (int s = 0; s < num_splits; ++s) m_all = fmaxf(m_all, partial_ml[(slot0 + s * stride) * 2]);
  float l_all = 0.0f, acc = 0.0f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = partial_ml[(slot0 + s * stride) * 2];
    const float w = ms == -INFINITY ? 0.0f : exp2f(ms - m_all);
    if (w > 0.0f) {  // a part without keys leaves no rows behind, only its (-inf, 0)
      l_all += partial_ml[(slot0 + s * stride) * 2 + 1] * w;
      acc += partial_o[(slot0 + s * stride) * D + threadIdx.x] * w;
    }
  }
  out[(size_t)token * out_stride + (size_t)head * D + threadIdx.x] =
      __float2bfloat16_rn(l_all > 0.0f ? acc / l_all : 0.0f);
}

static int page_shift_of(int page_size) {
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  return (1 << shift) == page_size ? shift : -1;
}

static int check_common(const void* q, long long q_stride, const void* out, long long out_stride,
                        int head_dim, int num_heads, int num_kv_heads, int page_size) {
  if (head_dim != 64 && head_dim != 128) return TS_ERR_SIZE;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads) return TS_ERR_SIZE;
  if (page_shift_of(page_size) < 0) return TS_ERR_SIZE;
  if (((uintptr_t)q & 3) || ((uintptr_t)out & 3) || (q_stride & 1) || (out_stride & 1)) return TS_ERR_ALIGN;
  return 0;
}

// Steps with prompts in them.  max_tiles: an upper bound of sum over requests of
// ceil(query_len / tokens_per_tile), tokens_per_tile = 64 / (num_heads / num_kv_heads).
TS_EXPORT int ts_flash_prefill(const void* q, long long q_stride, void* out, long long out_stride,
                               const void* k_pages, const void* v_pages, const int* block_table,
                               int table_stride, const int* query_start_loc, const int* context_lens,
                               int num_seqs, int max_tiles, int page_size, int num_heads,
                               int num_kv_heads, int head_dim, int window, float scale,
                               cudaStream_t stream) {
  if (num_seqs <= 0 || max_tiles <= 0) return 0;
  const int bad = check_common(q, q_stride, out, out_stride, head_dim, num_heads, num_kv_heads, page_size);
  if (bad) return bad;
  if (num_heads / num_kv_heads > FLASH_WARPS * 16) return TS_ERR_SIZE;
  if (num_kv_heads > 65535) return TS_ERR_SIZE;
  if (!(scale > 0.0f)) return TS_ERR_ARGUMENT;  // the running maximum is kept in unscaled units
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(max_tiles, num_kv_heads);
  const int shift = page_shift_of(page_size);
  const size_t smem = (size_t)4 * TILE_N * head_dim * sizeof(bf16);
  if (head_dim == 128) {
    cudaFuncSetAttribute(flash_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch(flash_prefill_kernel<128>, dim3(grid), dim3(FLASH_THREADS), smem, stream, 
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages, (const bf16*)v_pages,
        block_table, table_stride, query_start_loc, context_lens, num_seqs, shift, num_heads, num_kv_heads,
        window, scale_log2);
  } else {
    ts_launch(flash_prefill_kernel<64>, dim3(grid), dim3(FLASH_THREADS), smem, stream, 
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages, (const bf16*)v_pages,
        block_table, table_stride, query_start_loc, context_lens, num_seqs, shift, num_heads, num_kv_heads,
        window, scale_log2);
  }
  return ts_launch_status();
}

// Bytes of scratch a decode launch needs for (num_tokens, num_heads, num_splits, head_dim):
// partial_o then partial_ml, both fp32.
TS_EXPORT long long ts_flash_decode_scratch_floats(int num_tokens, int num_heads, int num_splits, int head_dim) {
  if (num_splits <= 1) return 0;
  return (long long)num_tokens * num_heads * num_splits * (head_dim + 2);
}

template <int D>
static int launch_decode(const bf16* q, long long q_stride, bf16* out, long long out_stride,
                         const bf16* k_pages, const bf16* v_pages, const int* block_table,
                         int table_stride, const int* seq_of_token, const int* positions,
                         int num_tokens, int shift, int num_heads, int num_kv_heads, int window,
                         float scale_log2, int num_splits, float* scratch, bool cluster, int* status,
                         cudaStream_t stream) {
  const size_t kv_smem = (size_t)FLASH_WARPS * DECODE_STAGES * 16 * D * sizeof(bf16);
  const size_t join_smem = (size_t)(FLASH_WARPS + 1) * 16 * (D + 2) * sizeof(float);  // the warps' join area, then the block's partials
  const size_t smem = kv_smem > join_smem ? kv_smem : join_smem;
  if (cluster) {
    // one cluster per (kv head, request): its blocks are the splits, joined over distributed shared memory
    cudaFuncSetAttribute(flash_decode_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ts_launch_cluster(flash_decode_kernel<D, true>, dim3(num_splits, num_kv_heads, num_tokens), dim3(FLASH_THREADS), smem,
                      stream, num_splits, q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride,
                      seq_of_token, positions, shift, num_heads, num_kv_heads, window, scale_log2, num_splits,
                      (float*)nullptr, (float*)nullptr, status);
    return ts_launch_status();
  }
  cudaFuncSetAttribute(flash_decode_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  float* partial_o = scratch;
  float* partial_ml = scratch ? scratch + (size_t)num_tokens * num_heads * num_splits * D : nullptr;
  dim3 grid(num_splits, num_kv_heads, num_tokens);
  ts_launch(flash_decode_kernel<D, false>, dim3(grid), dim3(FLASH_THREADS), smem, stream, 
      q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride, seq_of_token, positions,
      shift, num_heads, num_kv_heads, window, scale_log2, num_splits, partial_o, partial_ml, status);
  int code = ts_launch_status();
  if (code || num_splits == 1) return code;
  dim3 join_grid(num_heads, num_tokens);
  ts_launch(flash_decode_join_kernel<D>, dim3(join_grid), dim3(D), 0, stream, out, out_stride, seq_of_token, num_heads,
            num_splits, (const float*)partial_o, (const float*)partial_ml, (const int*)nullptr, (const int*)nullptr);
  return ts_launch_status();
}

// Decode steps (every token is its request's only query).  scratch: fp32, at least
// ts_flash_decode_scratch_floats(...) long when num_splits > DECODE_CLUSTER_MAX (fewer splits are
// joined inside a thread-block cluster and need none); its contents are dead after the call.
static int flash_decode_checked(const void* q, long long q_stride, void* out, long long out_stride,
                                const void* k_pages, const void* v_pages, const int* block_table,
                                int table_stride, const int* seq_of_token, const int* positions,
                                int num_tokens, int page_size, int num_heads, int num_kv_heads,
                                int head_dim, int window, float scale, int num_splits, float* scratch,
                                bool allow_cluster, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int bad = check_common(q, q_stride, out, out_stride, head_dim, num_heads, num_kv_heads, page_size);
  if (bad) return bad;
  if (num_heads / num_kv_heads > 16) return TS_ERR_SIZE;
  if (((uintptr_t)q & 15) || (q_stride & 7)) return TS_ERR_ALIGN;  // queries are read 16 bytes at a time
  if (num_splits < 1 || num_splits > 65535 || num_kv_heads > 65535 || num_tokens > 65535) return TS_ERR_SIZE;
  // two to DECODE_CLUSTER_MAX splits are joined inside a cluster and need no scratch
  const bool cluster = allow_cluster && num_splits >= 2 && num_splits <= DECODE_CLUSTER_MAX;
  if (num_splits > 1 && !cluster && (scratch == nullptr || ((uintptr_t)scratch & 15))) return TS_ERR_ARGUMENT;
  const float scale_log2 = scale * 1.4426950408889634f;
  const int shift = page_shift_of(page_size);
  if (head_dim == 128)
    return launch_decode<128>((const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages,
                              (const bf16*)v_pages, block_table, table_stride, seq_of_token, positions,
                              num_tokens, shift, num_heads, num_kv_heads, window, scale_log2, num_splits,
                              scratch, cluster, status, stream);
  return launch_decode<64>((const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages,
                           (const bf16*)v_pages, block_table, table_stride, seq_of_token, positions,
                           num_tokens, shift, num_heads, num_kv_heads, window, scale_log2, num_splits,
                           scratch, cluster, status, stream);
}

TS_EXPORT int ts_flash_decode(const void* q, long long q_stride, void* out, long long out_stride,
                              const void* k_pages, const void* v_pages, const int* block_table,
                              int table_stride, const int* seq_of_token, const int* positions,
                              int num_tokens, int page_size, int num_heads, int num_kv_heads,
                              int head_dim, int window, float scale, int num_splits, float* scratch,
                              int* status, cudaStream_t stream) {
  return flash_decode_checked(q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride,
                              seq_of_token, positions, num_tokens, page_size, num_heads, num_kv_heads, head_dim,
                              window, scale, num_splits, scratch, true, status, stream);
}

// ---- the TMA-fed decode kernel's host side -------------------------------------------------------
typedef CUresult (*DtmaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static DtmaEncodeFn dtma_encode_fn() {
  static DtmaEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = (DtmaEncodeFn)ptr;
  }
  return fn;
}

// The pool of one layer seen as a matrix: one row per (page, slot), kv_heads * head_dim columns.
static int dtma_make_map(CUtensorMap* map, const void* pages, long long rows, long long cols, int box_rows) {
  DtmaEncodeFn encode = dtma_encode_fn();
  if (encode == nullptr) return TS_ERR_ARGUMENT;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  const CUresult res = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box,
                              elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return res == CUDA_SUCCESS ? 0 : TS_ERR_ARGUMENT;
}

// The launches of a checked call, for one head size.
template <int D, bool FUSED>
static int flash_decode_tma_launch(const CUtensorMap& map_k, const CUtensorMap& map_v, const void* q, long long q_stride,
                                   void* out, long long out_stride, const int* block_table, int table_stride,
                                   const int* seq_of_token, const int* positions, int num_tokens, int shift, int box_rows,
                                   long long rows, int num_heads, int num_kv_heads, int window, float scale_log2,
                                   int num_splits, float* partial_o, float* partial_ml, int* status,
                                   const DecodeFusion& fusion, bool cluster, const DecodeItems& items, int num_items,
                                   cudaStream_t stream) {
  const bool listed = items.item_token != nullptr;
  const dim3 grid = listed ? dim3(num_items, num_kv_heads, 1) : dim3(num_splits, num_kv_heads, num_tokens);
  if (cluster) {
    cudaFuncSetAttribute(flash_decode_tma_kernel<D, true, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, DTMA_SMEM(D));
    ts_launch_cluster(flash_decode_tma_kernel<D, true, FUSED>, grid, dim3(DTMA_THREADS), DTMA_SMEM(D), stream, num_splits,
                      map_k, map_v, (const bf16*)q, q_stride, (bf16*)out, out_stride, block_table, table_stride,
                      seq_of_token, positions, shift, box_rows, (int)rows, num_heads, num_kv_heads, window, scale_log2,
                      num_splits, (float*)nullptr, (float*)nullptr, status, fusion, items);
    return ts_launch_status();
  }
  cudaFuncSetAttribute(flash_decode_tma_kernel<D, false, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, DTMA_SMEM(D));
  ts_launch(flash_decode_tma_kernel<D, false, FUSED>, grid, dim3(DTMA_THREADS), DTMA_SMEM(D), stream, map_k, map_v,
            (const bf16*)q, q_stride, (bf16*)out, out_stride, block_table, table_stride, seq_of_token, positions, shift,
            box_rows, (int)rows, num_heads, num_kv_heads, window, scale_log2, num_splits, partial_o, partial_ml, status,
            fusion, items);
  const int code = ts_launch_status();
  if (code || (num_splits == 1 && !listed)) return code;
  ts_launch(flash_decode_join_kernel<D>, dim3(num_heads, num_tokens), dim3(D), 0, stream, (bf16*)out, out_stride,
            seq_of_token, num_heads, num_splits, (const float*)partial_o, (const float*)partial_ml, items.parts_of,
            items.first_item);
  return ts_launch_status();
}

// Decode steps with head size 64 or 128 (the form that encodes and appends itself: 128 only) and
// pages of 4 to 2^30 tokens (a power of two), keys and values fetched by TMA.  Splits and
// scratch as for ts_flash_decode; num_pages is the pool's size.
template <bool FUSED>
static int flash_decode_tma_checked(const void* q, long long q_stride, void* out, long long out_stride,
                                    const void* k_pages, const void* v_pages, long long num_pages,
                                    const int* block_table, int table_stride, const int* seq_of_token,
                                    const int* positions, int num_tokens, int page_size, int num_heads,
                                    int num_kv_heads, int head_dim, int window, float scale, int num_splits,
                                    float* scratch, int* status, const DecodeFusion& fusion, bool allow_cluster,
                                    const DecodeItems& items, int num_items, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int bad = check_common(q, q_stride, out, out_stride, head_dim, num_heads, num_kv_heads, page_size);
  if (bad) return bad;
  if ((head_dim != 128 && (FUSED || head_dim != 64)) || page_size < 4) return TS_ERR_SIZE;
  if (num_heads / num_kv_heads > 16) return TS_ERR_SIZE;
  if (((uintptr_t)q & 3) || (q_stride & 1)) return TS_ERR_ALIGN;
  if (((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15)) return TS_ERR_ALIGN;
  if (num_splits < 1 || num_splits > 65535 || num_kv_heads > 65535 || num_tokens > 65535) return TS_ERR_SIZE;
  const bool listed = items.item_token != nullptr;
  if (listed && (num_items < 1 || num_items > 65535 || !items.item_part || !items.parts_of || !items.first_item))
    return TS_ERR_ARGUMENT;
  const bool cluster = !listed && allow_cluster && num_splits >= 2 && num_splits <= DECODE_CLUSTER_MAX;
  if ((num_splits > 1 || listed) && !cluster && (scratch == nullptr || ((uintptr_t)scratch & 15))) return TS_ERR_ARGUMENT;
  const long long rows = num_pages * page_size;
  if (rows <= 0 || rows >= (1ll << 31) - 256) return TS_ERR_SIZE;
  const int box_rows = page_size < DTMA_KEYS ? page_size : DTMA_KEYS;
  CUtensorMap map_k, map_v;
  int code = dtma_make_map(&map_k, k_pages, rows, (long long)num_kv_heads * head_dim, box_rows);
  if (code) return code;
  code = dtma_make_map(&map_v, v_pages, rows, (long long)num_kv_heads * head_dim, box_rows);
  if (code) return code;
  const float scale_log2 = scale * 1.4426950408889634f;
  const int shift = page_shift_of(page_size);
  float* partial_o = scratch;
  // scratch: the partial rows of every slot, then their (max, sum): [tokens, heads, splits], or [items, heads]
  const size_t slots = listed ? (size_t)num_items * num_heads : (size_t)num_tokens * num_heads * num_splits;
  float* partial_ml = scratch ? scratch + slots * head_dim : nullptr;
  if (head_dim == 128)
    return flash_decode_tma_launch<128, FUSED>(map_k, map_v, q, q_stride, out, out_stride, block_table, table_stride,
                                               seq_of_token, positions, num_tokens, shift, box_rows, rows, num_heads,
                                               num_kv_heads, window, scale_log2, num_splits, partial_o, partial_ml, status,
                                               fusion, cluster, items, num_items, stream);
  if constexpr (!FUSED)
    return flash_decode_tma_launch<64, false>(map_k, map_v, q, q_stride, out, out_stride, block_table, table_stride,
                                              seq_of_token, positions, num_tokens, shift, box_rows, rows, num_heads,
                                              num_kv_heads, window, scale_log2, num_splits, partial_o, partial_ml, status,
                                              fusion, cluster, items, num_items, stream);
  return TS_ERR_SIZE;
}

TS_EXPORT int ts_flash_decode_tma(const void* q, long long q_stride, void* out, long long out_stride,
                                  const void* k_pages, const void* v_pages, long long num_pages,
                                  const int* block_table, int table_stride, const int* seq_of_token,
                                  const int* positions, int num_tokens, int page_size, int num_heads,
                                  int num_kv_heads, int head_dim, int window, float scale, int num_splits,
                                  float* scratch, int* status, cudaStream_t stream) {
  DecodeFusion none;
  memset(&none, 0, sizeof(none));
  return flash_decode_tma_checked<false>(q, q_stride, out, out_stride, k_pages, v_pages, num_pages, block_table,
                                         table_stride, seq_of_token, positions, num_tokens, page_size, num_heads,
                                         num_kv_heads, head_dim, window, scale, num_splits, scratch, status, none, true,
                                         DecodeItems{nullptr, nullptr, nullptr, nullptr}, 0, stream);
}

// The same with a work list instead of one number of parts for every token (see DecodeItems):
// item_token / item_part hold num_items items (the grid), parts_of / first_item one entry per
// token; scratch holds num_items * num_heads * (head_dim + 2) floats.  A token with one part
// writes its output row itself, the others are joined by the second kernel.
TS_EXPORT int ts_flash_decode_tma_items(const void* q, long long q_stride, void* out, long long out_stride,
                                        const void* k_pages, const void* v_pages, long long num_pages,
                                        const int* block_table, int table_stride, const int* seq_of_token,
                                        const int* positions, int num_tokens, int page_size, int num_heads,
                                        int num_kv_heads, int head_dim, int window, float scale,
                                        const int* item_token, const int* item_part, const int* parts_of,
                                        const int* first_item, int num_items, float* scratch, int* status,
                                        cudaStream_t stream) {
  DecodeFusion none;
  memset(&none, 0, sizeof(none));
  return flash_decode_tma_checked<false>(q, q_stride, out, out_stride, k_pages, v_pages, num_pages, block_table,
                                         table_stride, seq_of_token, positions, num_tokens, page_size, num_heads,
                                         num_kv_heads, head_dim, window, scale, 1, scratch, status, none, false,
                                         DecodeItems{item_token, item_part, parts_of, first_item}, num_items, stream);
}

// The same, with the step before attention done by the kernel itself (see DecodeFusion): qkv is
// the raw product [tokens, qkv_stride] (query heads, key heads, value heads), bias fp32 or null,
// inv_freq fp32 [rotary_dim / 2]; the token's key and value are appended to the pages when
// write_kv is set.  Nothing of qkv is changed.  Without allow_cluster two to DECODE_CLUSTER_MAX
// splits also meet in scratch (which must then be given) and are joined by the second kernel.
TS_EXPORT int ts_flash_decode_tma_fused(const void* qkv, long long qkv_stride, const float* bias, const float* inv_freq,
                                        int rotary_dim, float factor, int write_kv, void* out, long long out_stride,
                                        void* k_pages, void* v_pages, long long num_pages, const int* block_table,
                                        int table_stride, const int* seq_of_token, const int* positions,
                                        int num_tokens, int page_size, int num_heads, int num_kv_heads, int head_dim,
                                        int window, float scale, int num_splits, float* scratch, int* status,
                                        int allow_cluster, cudaStream_t stream) {
  if (rotary_dim < 0 || rotary_dim > 128 || (rotary_dim & 1) || (rotary_dim > 0 && inv_freq == nullptr)) return TS_ERR_SIZE;
  if (!(factor > 0.0f)) return TS_ERR_ARGUMENT;
  if (qkv_stride < (long long)(num_heads + 2 * num_kv_heads) * 128) return TS_ERR_SIZE;
  DecodeFusion fusion;
  fusion.qkv = (const bf16*)qkv;
  fusion.qkv_stride = qkv_stride;
  fusion.bias = bias;
  fusion.inv_freq = inv_freq;
  fusion.rotary_dim = rotary_dim;
  fusion.factor = factor;
  fusion.k_pages = (bf16*)k_pages;
  fusion.v_pages = (bf16*)v_pages;
  fusion.write_kv = write_kv;
  return flash_decode_tma_checked<true>(qkv, qkv_stride, out, out_stride, k_pages, v_pages, num_pages, block_table,
                                        table_stride, seq_of_token, positions, num_tokens, page_size, num_heads,
                                        num_kv_heads, head_dim, window, scale, num_splits, scratch, status, fusion,
                                        allow_cluster != 0, DecodeItems{nullptr, nullptr, nullptr, nullptr}, 0, stream);
}

// ---------------------------------------------------------------------------------------------
// ts_flash_decode_static: the decode kernel for callers that cannot allocate device memory.
// Declared and documented in attention_bf16_static.h; it has no counterpart in the reference.
//
// The partial results of the splits live in the file-scope array below instead of a buffer
// from the caller.  Host code cannot pass the array's name to a kernel: on the host that name
// is only a handle, not a device address.  The address is asked for once per device with
// cudaGetSymbolAddress, with that device current, and kept in a table indexed by device.
// ---------------------------------------------------------------------------------------------
#define TS_STATIC_SCRATCH_FLOATS (1 << 20)  // 4 MiB, held by every device that loads this library
#define TS_STATIC_MAX_DEVICES 64
#define TS_ERR_STATIC_SCRATCH (-5)

static __device__ __align__(256) float ts_static_decode_scratch[TS_STATIC_SCRATCH_FLOATS];
static float* ts_static_decode_scratch_address[TS_STATIC_MAX_DEVICES];

TS_EXPORT long long ts_flash_decode_static_capacity_floats() { return TS_STATIC_SCRATCH_FLOATS; }

TS_EXPORT int ts_flash_decode_static(const void* q, long long q_stride, void* out, long long out_stride,
                                     const void* k_pages, const void* v_pages, const int* block_table,
                                     int table_stride, const int* seq_of_token, const int* positions,
                                     int num_tokens, int page_size, int num_heads, int num_kv_heads,
                                     int head_dim, int window, float scale, int num_splits,
                                     cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (num_splits < 1) return TS_ERR_SIZE;
  const long long need = ts_flash_decode_scratch_floats(num_tokens, num_heads, num_splits, head_dim);
  if (need > TS_STATIC_SCRATCH_FLOATS) return TS_ERR_STATIC_SCRATCH;
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return (int)err;
  if (device < 0 || device >= TS_STATIC_MAX_DEVICES) return TS_ERR_ARGUMENT;
  float* scratch = ts_static_decode_scratch_address[device];
  if (scratch == nullptr) {
    // first call on this device: look the array's device address up (no allocation happens here)
    err = cudaGetSymbolAddress((void**)&scratch, ts_static_decode_scratch);
    if (err != cudaSuccess) return (int)err;
    if (scratch == nullptr) return TS_ERR_ARGUMENT;
    ts_static_decode_scratch_address[device] = scratch;
  }
  // always the scratch path: the splits meet in the static array, never in a cluster
  return flash_decode_checked(q, q_stride, out, out_stride, k_pages, v_pages, block_table, table_stride,
                              seq_of_token, positions, num_tokens, page_size, num_heads, num_kv_heads, head_dim,
                              window, scale, num_splits, scratch, false, nullptr, stream);
}
