// Paged attention for steps with prompts in them on the fifth-generation tensor cores:
// S = Q K^T and O += P V are tcgen05.mma with both accumulators in tensor memory, keys and values
// come straight from the paged cache by TMA.  bfloat16, head size 128.
//
// A block owns 128 rows of one kv head: (query token, query head of the group) pairs, so the
// heads of a group share every key tile (18 tokens x 7 heads for Qwen2-7B), and walks that
// request's keys in tiles of 64 through its block table.  Two blocks share an SM (98 KB of
// shared memory and 256 columns of tensor memory each): while one is in its softmax the other
// has the tensor cores, which a single block, bound by the latency of its softmax chain,
// keeps busy only a fifth of the time.
//   warp 9             producer: one lane per page of the tile looks its page up and issues the TMA
//                      loads (one box per page and 64-dim half, 128-byte swizzle; a page that
//                      was given back or lies past the table is fetched from an out-of-range
//                      row, which TMA fills with zeros); keys have two stages and are fetched a
//                      tile ahead, values one stage that is refilled as soon as O has read it;
//   warp 8, one lane   MMA issuer: per tile 8 MMAs for S (M 128, N 64 keys, K 16 dims each) into
//                      one of two S buffers and 8 for O (M 128, N 64 dims, K 16 keys each, V
//                      read as an MN-major operand); S of the next tile is started before P of
//                      this tile is waited for; tcgen05.commit on mbarriers tells the others;
//   warps 0..7         softmax: row r = TMEM lane r belongs to threads r and 128 + r, each with
//                      32 of the tile's 64 scores: they read them from tensor memory, mask
//                      (causal, window), exchange their maxima through shared memory (an
//                      mbarrier per pair of warps), keep the running maximum and sum in fp32,
//                      rescale their half of the O row in tensor memory when the maximum moved
//                      far, write their half of the P row as bfloat16 into the swizzled
//                      shared-memory tile the second MMA reads, and at the end normalise and
//                      store their half of the output row.
//
// Tried and dropped: sharing a long row tile between the two blocks of a cluster (lower and upper
// half of the keys, merged over distributed shared memory) to shorten the longest blocks.  A
// cluster keeps both of its slots until both blocks are done, so every row tile that is not
// shared idles a slot (2,048 tokens: 122 us with no tile shared, 93 us with all shared, against
// 85 us without clusters; 8,192 tokens: 767 us against 685 us).
//
// Tried and dropped too: the same sharing between two ordinary blocks that meet in scratch memory
// (each leaves its unnormalised rows and draws a ticket; the second adds the other's to its own),
// which holds no slot idle.  Correct and bit-stable, but slower wherever it applied to a prompt of
// 1,024 tokens or more (2,048 tokens: 86 us with tiles of 12 or more key tiles shared, 84 us from
// 20, against 75 us unshared): with that many row tiles the length of the longest block is not
// what bounds the step.  It is with few row tiles (a portion of a prompt late in a long context):
// there the keys of every tile are cut into parts, see SPLIT below and atc_parts().
//
// Tried and dropped: one lane per warp waiting on (and arriving at) the row threads' mbarriers, the
// others following through a shuffle.  The trace shows 400 to 600 cycles per wait with all lanes
// in try_wait even when the phase is long complete, yet every elected-lane form was slower
// overall (2,048 tokens: 114 to 124 us against 85 us; with try_wait, with a test_wait spin, with
// a short suspend hint): the waits of the other kind grew by more than these shrank.
//
// Tried and dropped too: the two warps of a row pair meeting at a named hardware barrier of their own
// (bar.red.and over 64 threads, which also carries "nobody has given up", one meeting a tile with
// the exchanged numbers in two buffers) instead of the two mbarriers: correct, and slower
// (2,048 tokens: 83.5 us against 74; 8,192: 813 against 688).
//
// Tried and dropped: a second form of the kernel after the published Blackwell attention designs: a
// block alone on its multiprocessor with TWO row tiles that take turns on the tensor cores, key
// tiles of 128, one softmax thread per row with all 128 scores in registers (no exchange between
// threads), and P written back into tensor memory over the scores (tcgen05.st of packed bfloat16
// pairs, column c = keys 2c and 2c + 1) and read from there as the A operand of the O product
// (tcgen05.mma with [a_taddr]: exact in a one-block probe and in the kernel's tests).  Correct on
// every shape of the tests, bit-stable, and slower: 2,048 tokens 92 us against 70, 8,192 944
// against 648, 16,384 3,553 against 2,404 (542 against 800 TFLOP/s).  A trace of its softmax
// threads: per 128-key step 2,400 to 3,100 cycles waiting for the scores, 700 to 900 for one round
// of tcgen05.ld + wait, 5,200 to 5,900 for maximum, exponentials, packing and the store: eight
// softmax warps a multiprocessor (two per scheduler) do not hide the latency of their own chains,
// where the two blocks of the kernel above bring sixteen.  Reading the scores twice (the maximum
// first, 32 at a time, to keep fewer registers) was worse still (344 TFLOP/s): every round of
// tcgen05.ld + wait costs 700 to 1,200 cycles while the tensor cores run the other tile.  It
// would take what the published designs add on top (exponentials partly as polynomials on the
// FMA pipes, a correction warp group, more stages).
//
// Every mbarrier wait is bounded; a wait that runs out raises bit 32 of *status, the block stops,
// frees its tensor memory and returns.  No cluster, no multicast.
// Replaces the reference's per-sequence gather + SDPA (src/turboserve/engine/model/
// attention.py:184-209).
#include <cuda.h>

#include "common.cuh"

#define ATC_D 128
#define ATC_ROWS 128
#define ATC_KEYS 64                           // keys per tile
#define ATC_SPLIT 2                           // threads per row
#define ATC_COLS (ATC_KEYS / ATC_SPLIT)       // scores (columns of S, of P) per thread and tile
#define ATC_OCOLS (ATC_D / ATC_SPLIT)         // dims of Q and O per thread
#define ATC_ROW_THREADS (128 * ATC_SPLIT)
#define ATC_ROW_WARPS (4 * ATC_SPLIT)
#define ATC_THREADS (ATC_ROW_THREADS + 64)    // softmax warps, the MMA issuer's warp, the producer warp
#define ATC_WAIT_LIMIT (1 << 24)
#define ATC_Q_HALF 16384                      // [128 rows x 64 dims] bf16
#define ATC_KV_HALF 8192                      // [64 keys x 64 dims] bf16
#define ATC_Q_OFF 0
#define ATC_P_OFF 32768                       // [128 rows x 64 keys] bf16, one buffer
#define ATC_K_OFF 49152                       // two stages of keys (two dim halves each)
#define ATC_V_OFF 81920                       // one stage of values
#define ATC_TILES_BYTES 98304
#ifndef ATC_SLACK
#define ATC_SLACK 1024  // room to round the tiles' start up to 1,024 bytes; the kernel checks that it was enough
#endif
#define ATC_SMEM (ATC_TILES_BYTES + ATC_SLACK)
#define ATC_TMEM_COLS 256                     // S: two buffers of 64 columns; O: 128 columns
#define ATC_PART_FLOATS (ATC_ROWS * ATC_D + 2 * ATC_ROWS)  // what a block of a split tile leaves: O rows, then (m, l) per row
#define ATC_MAX_PARTS 8
#define ATC_TWO_WAVE_TILES 128                // key tiles from which two parts pay with a few more row tiles than multiprocessors
#define ATC_MIN_PART_TILES 4                  // a part is worth a block from this many 64-key tiles

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ unsigned atc_smem(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void atc_mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void atc_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void atc_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool atc_try_wait(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool atc_wait(unsigned bar, unsigned parity, volatile int* failed) {
  for (int i = 0; i < ATC_WAIT_LIMIT; ++i) {
    if (atc_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023 && *failed) return false;
  }
  return false;
}
__device__ __forceinline__ void atc_tma_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle, groups of 8 rows 1024 bytes apart.  The
// leading-dimension field is not relied on: every operand block here is one swizzle span wide.
__device__ __forceinline__ unsigned long long atc_desc(unsigned addr) {
  unsigned long long d = 0;
  d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
  d |= (unsigned long long)1 << 16;
  d |= (unsigned long long)(1024 >> 4) << 32;
  d |= (unsigned long long)1 << 46;
  d |= (unsigned long long)2 << 61;
  return d;
}
__device__ __forceinline__ void atc_mma(unsigned d_tmem, unsigned long long a, unsigned long long b, unsigned idesc,
                                        unsigned accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void atc_commit(unsigned bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void atc_ld32(unsigned taddr, float (&v)[32]) {
  unsigned r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void atc_ld64(unsigned taddr, float (&v)[64]) {
  unsigned r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void atc_ld_cols(unsigned taddr, float (&v)[64]) { atc_ld64(taddr, v); }
__device__ __forceinline__ void atc_ld_cols(unsigned taddr, float (&v)[32]) { atc_ld32(taddr, v); }
__device__ __forceinline__ float atc_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void atc_st32(unsigned taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
        "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
        "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ unsigned atc_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

template <bool SPLIT>
__global__ void __launch_bounds__(ATC_THREADS, 2)
flash_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                        long long out_stride, const int* __restrict__ block_table, int table_stride,
                        const int* __restrict__ query_start_loc, const int* __restrict__ context_lens,
                        int num_seqs, int page_shift, int box_rows, int total_rows, int num_heads,
                        int num_kv_heads, int window, float scale_log2, int num_parts,
                        float* __restrict__ part_scratch, int* __restrict__ status) {
  pdl_wait();
  pdl_trigger<8>();
  extern __shared__ unsigned char atc_raw[];
  __shared__ __align__(8) unsigned long long bars[18];
  __shared__ unsigned tmem_slot;
  __shared__ int failed;
  __shared__ int s_seq, s_tile;
  __shared__ float row_pair[ATC_SPLIT][ATC_ROWS];  // [part][row]: what the threads of a row tell each other

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = num_heads / num_kv_heads;
  const int tokens_per_tile = ATC_ROWS / group;
  const unsigned base = (atc_smem(atc_raw) + 1023u) & ~1023u;
  if (base + ATC_TILES_BYTES > atc_smem(atc_raw) + ATC_SMEM) {  // the same for every thread: nothing has been set up yet
    if (threadIdx.x == 0 && status) atomicOr(status, 32);
    return;
  }
  const unsigned q_s = base + ATC_Q_OFF, p_s = base + ATC_P_OFF, k_s = base + ATC_K_OFF, v_s = base + ATC_V_OFF;
  // barriers: per key stage "landed" and "read"; "values landed", "values read"; per S buffer
  // "scores ready"; "P written" (all row threads); "O updated from it"
  const unsigned k_full = atc_smem(&bars[0]), k_empty = atc_smem(&bars[2]);
  const unsigned v_full = atc_smem(&bars[4]), v_empty = atc_smem(&bars[5]);
  const unsigned s_full = atc_smem(&bars[6]), p_ready = atc_smem(&bars[8]), o_full = atc_smem(&bars[9]);
  // per pair of warps that share 32 rows: "both have written their number", "both have read the other's"
  const unsigned pair_written = atc_smem(&bars[10 + (warp & 3)]), pair_read = atc_smem(&bars[14 + (warp & 3)]);

  if (threadIdx.x == 0) {
    failed = 0;
    for (int i = 0; i < 10; ++i) atc_mbar_init(atc_smem(&bars[i]), i == 8 ? ATC_ROW_THREADS : 1);
    for (int i = 10; i < 18; ++i) atc_mbar_init(atc_smem(&bars[i]), 32 * ATC_SPLIT);  // the warps that share 32 rows
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // longest tiles first: the last tiles of a request get the lowest block indices
    // block index = (row tile, kv head), the head fastest: the longest tiles of every head start first.
    // (With the head as a second grid dimension the last head's long tiles started when the others'
    // short ones were done, and the kernel ended on them: 88 instead of 75 us for a 2,048-token prompt.)
    // (SPLIT: the parts of a tile's keys are the fastest index, one block each)
    int remaining = (SPLIT ? blockIdx.x / num_parts : blockIdx.x) / num_kv_heads, found = -1, tile = 0;
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
  if (!SPLIT && warp == ATC_ROW_WARPS) {  // (SPLIT: further down, once the part is known to have keys)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(atc_smem(&tmem_slot)), "r"((unsigned)ATC_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }

  const int kv_head = (SPLIT ? blockIdx.x / num_parts : blockIdx.x) % num_kv_heads;
  const int q_begin = query_start_loc[seq], q_len = query_start_loc[seq + 1] - q_begin;
  const int ctx = context_lens[seq];
  const int tok0 = s_tile * tokens_per_tile;
  const int tile_tokens = min(tokens_per_tile, q_len - tok0);
  const int pos0 = ctx - q_len + tok0;
  const int* table = block_table + (size_t)seq * table_stride;
  const int kv_first = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int kv_end = pos0 + tile_tokens;
  // SPLIT: this block takes one of num_parts runs of the tile's 64-key tiles (it may be empty) and
  // leaves its unnormalised rows in scratch memory; a second kernel adds the parts up.
  const int all_begin = kv_first / ATC_KEYS, all_end = (kv_end + ATC_KEYS - 1) / ATC_KEYS;
  const int per_part = SPLIT ? (all_end - all_begin + num_parts - 1) / num_parts : all_end - all_begin;
  const int tile_begin = SPLIT ? min(all_end, all_begin + (int)(blockIdx.x % num_parts) * per_part) : all_begin;
  const int tile_end = SPLIT ? min(all_end, tile_begin + per_part) : all_end;
  const int num_tiles = tile_end - tile_begin;
  if (SPLIT && num_tiles <= 0) {  // an empty part (the same for every thread; nothing is held yet): no keys, no weight
    if (threadIdx.x < ATC_ROWS)
      reinterpret_cast<float2*>(part_scratch + (size_t)blockIdx.x * ATC_PART_FLOATS + ATC_ROWS * ATC_D)[threadIdx.x] =
          make_float2(-INFINITY, 0.0f);
    return;
  }
  if (SPLIT && warp == ATC_ROW_WARPS) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(atc_smem(&tmem_slot)), "r"((unsigned)ATC_TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }

  // ---- Q rows to shared memory (row threads) ------------------------------------------------------
  int my_pos = -1, my_first = 0;
  bf16* my_out = nullptr;
  const int part = warp >> 2;  // row threads: which columns of the row (keys of S, dims of Q and O)
  if (warp < ATC_ROW_WARPS) {
    const int r = threadIdx.x & 127;
    const int tok = r / group, head = kv_head * group + r % group;
    const bool valid = tok < tile_tokens;
    if (valid) {
      my_pos = pos0 + tok;
      my_first = window > 0 ? max(0, my_pos - window + 1) : 0;
      my_out = out + (size_t)(q_begin + tok0 + tok) * out_stride + (size_t)head * ATC_D + part * ATC_OCOLS;
    }
    const bf16* q_row = q + (size_t)(q_begin + tok0 + tok) * q_stride + (size_t)head * ATC_D + part * ATC_OCOLS;
#pragma unroll
    for (int i = 0; i < ATC_OCOLS / 8; ++i) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (valid) v = *reinterpret_cast<const uint4*>(q_row + i * 8);
      const int c = part * (ATC_OCOLS / 8) + i;  // 16-byte chunk of the row: 8 per 64-dim half
      const unsigned dst = q_s + (c >> 3) * ATC_Q_HALF + r * 128 + (((c & 7) ^ (r & 7)) << 4);
      asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const unsigned tmem = tmem_slot;
  const unsigned tmem_o = tmem + 2 * ATC_KEYS;  // S buffers at columns 0 and 64, O behind them

  if (warp == ATC_ROW_WARPS + 1) {
    // ---- producer warp: one lane per box (a page, or 64 keys of a larger page) ----------------------
    const int page_size = 1 << page_shift;
    const int boxes = ATC_KEYS / box_rows;
    bool ok = true;
    auto box_row = [&](int j) -> int {  // the row of the pool this lane's box of tile j starts at
      int row = total_rows;             // out of range: the box is filled with zeros
      if (lane < boxes) {
        const int key = (tile_begin + j) * ATC_KEYS + lane * box_rows;
        if (key < kv_end && key + box_rows > kv_first) {
          const int page = table[key >> page_shift];
          if (page >= 0) row = page * page_size + (key & (page_size - 1));
          else if (status) atomicOr(status, 4);  // a page in reach of this tile is missing
        }
      }
      return row;
    };
    auto load_keys = [&](int j, int row) -> bool {  // two stages; a stage is free once the S product of tile j - 2 has read it
      const int st = j & 1;
      if (j >= 2 && !__all_sync(0xffffffffu, atc_wait(k_empty + 8 * st, ((j >> 1) - 1) & 1, &failed))) return false;
      if (lane == 0) atc_expect_tx(k_full + 8 * st, 2 * ATC_KV_HALF);
      __syncwarp();
      if (lane < boxes) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
          atc_tma_2d(k_s + st * 2 * ATC_KV_HALF + h * ATC_KV_HALF + lane * box_rows * 128, &map_k, kv_head * ATC_D + h * 64, row, k_full + 8 * st);
      }
      return true;
    };
    int row = box_row(0);
    ok = num_tiles == 0 || load_keys(0, row);
    for (int j = 0; j < num_tiles && ok; ++j) {
      // the keys of the next tile go first: its S product is started a tile ahead
      const int next_row = j + 1 < num_tiles ? box_row(j + 1) : total_rows;
      if (j + 1 < num_tiles) ok = load_keys(j + 1, next_row);
      // values: one stage, free once the O product of the tile before has read it
      if (ok && j >= 1) ok = __all_sync(0xffffffffu, atc_wait(v_empty, (j - 1) & 1, &failed));
      if (!ok) break;
      if (lane == 0) atc_expect_tx(v_full, 2 * ATC_KV_HALF);
      __syncwarp();
      if (lane < boxes) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
          atc_tma_2d(v_s + h * ATC_KV_HALF + lane * box_rows * 128, &map_v, kv_head * ATC_D + h * 64, row, v_full);
      }
      row = next_row;
    }
    if (!ok && lane == 0) {
      failed = 1;
      if (status) atomicOr(status, 32);
    }
  } else if (warp == ATC_ROW_WARPS) {
    if (lane == 0) {
      // ---- MMA issuer: S(j + 1) is started before P(j) is waited for, so the tensor cores work on
      // the next scores while the row threads are in the softmax of this tile ----------------------
      const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);  // M 128, N 64
      const unsigned idesc_pv = idesc | (1u << 16);                                                        // B MN-major
      auto issue_qk = [&](int j) -> bool {
        if (!atc_wait(k_full + 8 * (j & 1), (j >> 1) & 1, &failed)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const unsigned keys = k_s + (j & 1) * 2 * ATC_KV_HALF;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)  // 16 dims per step; dims 64.. live in the second half
          atc_mma(tmem + (j & 1) * ATC_KEYS, atc_desc(q_s + (kk >> 2) * ATC_Q_HALF + (kk & 3) * 32),
                  atc_desc(keys + (kk >> 2) * ATC_KV_HALF + (kk & 3) * 32), idesc, kk != 0);
        atc_commit(s_full + 8 * (j & 1));
        atc_commit(k_empty + 8 * (j & 1));
        return true;
      };
      bool ok = num_tiles == 0 || issue_qk(0);  // a part of a split tile may be empty
      for (int j = 0; j < num_tiles && ok; ++j) {
        if (j + 1 < num_tiles) ok = issue_qk(j + 1);
        ok = ok && atc_wait(p_ready, j & 1, &failed) && atc_wait(v_full, j & 1, &failed);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int kk = 0; kk < ATC_KEYS / 16; ++kk) {  // 16 keys per step
          const unsigned long long a = atc_desc(p_s + kk * 32);
#pragma unroll
          for (int h = 0; h < 2; ++h)   // two N = 64 products: dims 0..63 and 64..127
            atc_mma(tmem_o + h * 64, a, atc_desc(v_s + h * ATC_KV_HALF + kk * 2048), idesc_pv, (j | kk) != 0);
        }
        atc_commit(o_full);
        atc_commit(v_empty);
      }
      if (!ok) {
        failed = 1;
        if (status) atomicOr(status, 32);
      }
    }
  } else {
    // ---- row threads: softmax, P, O rescale, output -------------------------------------------------
    // Row r belongs to threads r and 128 + r (warps w and w + 4 reach the same 32 lanes of tensor
    // memory): each takes half of the tile's scores, of the columns of P and of the dims of O.  Per
    // tile they exchange one number, their maximum, through shared memory; their sums meet at the end.
    const int r = threadIdx.x & 127;
    const unsigned lane_base = (unsigned)((warp & 3) * 32) << 16;
    float m = -INFINITY;  // the maximum the exponentials are taken against (raw score units)
    float2 l2 = make_float2(0.0f, 0.0f);
    bool ok = true;
    for (int j = 0; j < num_tiles; ++j) {
      ok = __all_sync(0xffffffffu, atc_wait(s_full + 8 * (j & 1), (j >> 1) & 1, &failed));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int key0 = (tile_begin + j) * ATC_KEYS + part * ATC_COLS;
      const bool masked = key0 + ATC_COLS - 1 > my_pos || key0 < my_first;
      float v[ATC_COLS];
      atc_ld32(tmem + (j & 1) * ATC_KEYS + part * ATC_COLS + lane_base, v);
      if (masked) {
#pragma unroll
        for (int i = 0; i < ATC_COLS; ++i) {
          const int key = key0 + i;
          if (!(key <= my_pos && key >= my_first)) v[i] = -INFINITY;
        }
      }
      // four chains, not one of ATC_COLS dependent steps: the row threads are bound by latency
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int i = 0; i < ATC_COLS; i += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) mx4[e] = fmaxf(mx4[e], v[i + e]);
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      if (j > 0) {  // the other thread of the row has read the number of the tile before (long ago, as a rule)
        ok = __all_sync(0xffffffffu, atc_wait(pair_read, (j - 1) & 1, &failed));
        if (!ok) break;
      }
      row_pair[part][r] = mx;
      atc_arrive(pair_written);
      ok = __all_sync(0xffffffffu, atc_wait(pair_written, j & 1, &failed));
      if (!ok) break;
#pragma unroll
      for (int other = 0; other < ATC_SPLIT; ++other) mx = fmaxf(mx, row_pair[other][r]);
      atc_arrive(pair_read);
      // The reference maximum moves only when the new one is far above it (2^8 in the exponent):
      // until then the exponentials may exceed one, which fp32 sums and bfloat16 P hold easily,
      // and the O row in tensor memory needs no rescaling.
      float corr = 1.0f;
      const bool move = mx > m && (m == -INFINITY || (mx - m) * scale_log2 > 8.0f);
      if (move) {
        corr = atc_ex2((m - mx) * scale_log2);  // 0 for the first tile
        m = mx;
        l2.x *= corr;
        l2.y *= corr;
      }
      const float shift = m == -INFINITY ? 0.0f : -m * scale_log2;
      const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(shift, shift);
      unsigned packed[ATC_COLS / 2];
      float2 sums[4] = {l2, make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
      for (int i = 0; i < ATC_COLS / 2; ++i) {
        const float2 e = __ffma2_rn(make_float2(v[2 * i], v[2 * i + 1]), scale2, shift2);
        const float2 pr = make_float2(atc_ex2(e.x), atc_ex2(e.y));  // -inf -> 0
        sums[i & 3] = __fadd2_rn(sums[i & 3], pr);
        packed[i] = atc_pack(pr.x, pr.y);
      }
      l2 = __fadd2_rn(__fadd2_rn(sums[0], sums[1]), __fadd2_rn(sums[2], sums[3]));
      if (j > 0) {
        // the O product of the tile before has read P (one buffer) and completed O
        ok = __all_sync(0xffffffffu, atc_wait(o_full, (j - 1) & 1, &failed));
        if (!ok) break;
        if (__any_sync(0xffffffffu, move)) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
          for (int c = 0; c < ATC_OCOLS / 32; ++c) {
            float o[32];
            atc_ld32(tmem_o + part * ATC_OCOLS + lane_base + c * 32, o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] *= corr;
            atc_st32(tmem_o + part * ATC_OCOLS + lane_base + c * 32, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
#pragma unroll
      for (int i = 0; i < ATC_COLS / 8; ++i) {  // 16-byte chunks of 8 keys; a row of P is 8 chunks
        const int chunk = part * (ATC_COLS / 8) + i;
        const unsigned dst = p_s + r * 128 + ((chunk ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(packed[4 * i]), "r"(packed[4 * i + 1]),
                     "r"(packed[4 * i + 2]), "r"(packed[4 * i + 3]) : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      atc_arrive(p_ready);
    }
    if (ok && num_tiles > 0) {
      ok = __all_sync(0xffffffffu, atc_wait(o_full, (num_tiles - 1) & 1, &failed));
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    if (!ok && lane == 0) {
      failed = 1;
      if (status) atomicOr(status, 32);
    }
    // the threads of a row add their sums
    if (ok && num_tiles > 0) ok = __all_sync(0xffffffffu, atc_wait(pair_read, (num_tiles - 1) & 1, &failed));
    if (ok) {
      row_pair[part][r] = l2.x + l2.y;
      atc_arrive(pair_written);
      ok = __all_sync(0xffffffffu, atc_wait(pair_written, num_tiles & 1, &failed));
    }
    if (ok) {
      float l = 0.0f;
#pragma unroll
      for (int other = 0; other < ATC_SPLIT; ++other) l += row_pair[other][r];
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      if constexpr (SPLIT) {
        // rows against this block's own maximum; consecutive rows lie side by side in scratch
        float* mine = part_scratch + (size_t)blockIdx.x * ATC_PART_FLOATS;
        if (num_tiles > 0) {
#pragma unroll
          for (int c = 0; c < ATC_OCOLS / 32; ++c) {
            float o[32];
            atc_ld32(tmem_o + part * ATC_OCOLS + lane_base + c * 32, o);
#pragma unroll
            for (int i = 0; i < 8; ++i)
              reinterpret_cast<float4*>(mine)[(size_t)(part * (ATC_OCOLS / 4) + c * 8 + i) * ATC_ROWS + r] =
                  make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
          }
        }
        if (part == 0) reinterpret_cast<float2*>(mine + ATC_ROWS * ATC_D)[r] = make_float2(num_tiles > 0 ? m : -INFINITY, l);
      }
#pragma unroll
      for (int c = 0; c < ATC_OCOLS / 32; ++c) {
        if constexpr (SPLIT) break;
        float o[32];
        atc_ld32(tmem_o + part * ATC_OCOLS + lane_base + c * 32, o);
        if (my_out) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = atc_pack(o[8 * i] * inv, o[8 * i + 1] * inv);
            w.y = atc_pack(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
            w.z = atc_pack(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
            w.w = atc_pack(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
            *reinterpret_cast<uint4*>(my_out + c * 32 + i * 8) = w;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (failed && threadIdx.x == 0) {
    // copies that were issued may still be landing: give them a bounded while
    const unsigned landing[3] = {k_full, k_full + 8, v_full};
    for (int s = 0; s < 3; ++s)
      for (int i = 0; i < 4096 && !atc_try_wait(landing[s], 0) && !atc_try_wait(landing[s], 1); ++i) {}
  }
  if (warp == ATC_ROW_WARPS) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((unsigned)ATC_TMEM_COLS));
}

// Adds up the parts of split tiles: one block per (row tile, kv head), thread = (row, half of the
// dims) as in the kernel above; parts in index order, so the result does not depend on timing.
__global__ void __launch_bounds__(2 * ATC_ROWS)
flash_prefill_tc_merge_kernel(const float* __restrict__ part_scratch, int num_parts, bf16* __restrict__ out,
                              long long out_stride, const int* __restrict__ query_start_loc, int num_seqs,
                              int num_heads, int num_kv_heads, float scale_log2) {
  pdl_wait();
  __shared__ int s_seq, s_tile;
  const int group = num_heads / num_kv_heads;
  const int tokens_per_tile = ATC_ROWS / group;
  if (threadIdx.x == 0) {
    int remaining = blockIdx.x / num_kv_heads, found = -1, tile = 0;
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
  const int kv_head = blockIdx.x % num_kv_heads;
  const int q_begin = query_start_loc[seq], q_len = query_start_loc[seq + 1] - q_begin;
  const int tok0 = s_tile * tokens_per_tile;
  const int r = threadIdx.x & (ATC_ROWS - 1), half = threadIdx.x / ATC_ROWS;
  const int tok = r / group, head = kv_head * group + r % group;
  if (tok >= min(tokens_per_tile, q_len - tok0)) return;
  const float* base = part_scratch + (size_t)blockIdx.x * num_parts * ATC_PART_FLOATS;
  float w[ATC_MAX_PARTS], top = -INFINITY, l = 0.0f;
#pragma unroll
  for (int p = 0; p < ATC_MAX_PARTS; ++p) {
    w[p] = -INFINITY;
    if (p < num_parts) w[p] = __ldcg(reinterpret_cast<const float2*>(base + (size_t)p * ATC_PART_FLOATS + ATC_ROWS * ATC_D) + r).x;
    top = fmaxf(top, w[p]);
  }
#pragma unroll
  for (int p = 0; p < ATC_MAX_PARTS; ++p) {
    const float m = w[p];
    w[p] = m == -INFINITY ? 0.0f : exp2f((m - top) * scale_log2);
    if (p < num_parts && w[p] > 0.0f)
      l += __ldcg(reinterpret_cast<const float2*>(base + (size_t)p * ATC_PART_FLOATS + ATC_ROWS * ATC_D) + r).y * w[p];
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  bf16* dst = out + (size_t)(q_begin + tok0 + tok) * out_stride + (size_t)head * ATC_D + half * ATC_OCOLS;
#pragma unroll 2
  for (int c8 = 0; c8 < ATC_OCOLS / 8; ++c8) {
    float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int p = 0; p < ATC_MAX_PARTS; ++p) {
      if (p < num_parts && w[p] > 0.0f) {
        const float4* rows = reinterpret_cast<const float4*>(base + (size_t)p * ATC_PART_FLOATS);
        const float4 a = __ldcg(rows + (size_t)(half * (ATC_OCOLS / 4) + 2 * c8) * ATC_ROWS + r);
        const float4 b = __ldcg(rows + (size_t)(half * (ATC_OCOLS / 4) + 2 * c8 + 1) * ATC_ROWS + r);
        acc[0] += a.x * w[p]; acc[1] += a.y * w[p]; acc[2] += a.z * w[p]; acc[3] += a.w * w[p];
        acc[4] += b.x * w[p]; acc[5] += b.y * w[p]; acc[6] += b.z * w[p]; acc[7] += b.w * w[p];
      }
    }
    uint4 packed;
    packed.x = atc_pack(acc[0] * inv, acc[1] * inv);
    packed.y = atc_pack(acc[2] * inv, acc[3] * inv);
    packed.z = atc_pack(acc[4] * inv, acc[5] * inv);
    packed.w = atc_pack(acc[6] * inv, acc[7] * inv);
    *reinterpret_cast<uint4*>(dst + c8 * 8) = packed;
  }
}

// ---- host side ------------------------------------------------------------------------------------

typedef CUresult (*AtcEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static AtcEncodeFn atc_encode_fn() {
  static AtcEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      fn = (AtcEncodeFn)ptr;
  }
  return fn;
}

static int atc_num_sms() {
  static int sms = 0;
  if (sms == 0) {
    int device = 0;
    cudaGetDevice(&device);
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0) sms = 1;
  }
  return sms;
}

// The pool of one layer seen as a matrix: one row per (page, slot), kv_heads * head_dim columns.
static int atc_make_map(CUtensorMap* map, const void* pages, long long rows, long long cols, int box_rows) {
  AtcEncodeFn encode = atc_encode_fn();
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

// Few row tiles for the device (a portion of a prompt, late in a long context): each is a long
// chain of key tiles in one block while most multiprocessors idle.  Then the keys of every tile are
// cut into parts, one block each, and a second kernel adds the parts up.  How many parts, from what
// the host knows (an upper bound of the row tiles, the longest context): as many as keep all blocks
// on the device at once (two a multiprocessor), eight at most, four key tiles a part at least; and
// only with no more row tiles than multiprocessors, and when the step gets 15 % shorter by this
// estimate: a block alone on its multiprocessor takes about 1.3 us a key tile, one of two 1.9 us,
// 6 us go to a block's start and end and 6 us to the partial rows and the second kernel.
// (Measured, 28 heads on 4: 512 tokens at context 8,192 163 -> 128 us, 256 at 4,096 85 -> 51 us,
// 64 at 16,384 309 -> 60 us.)  With a few more row tiles than multiprocessors (up to 5/4 of them), two
// parts gain about 15 % from a context of 8,192 (40 heads on 8, 512 tokens: 221 -> 188 us; 441 -> 371
// us at 16,384), 6 % at 4,096 and lose at 1,512 (41 -> 57 us): two parts from 128 key tiles.  With
// more row tiles than that, whole tiles fill the device better (232 row tiles: 192 -> 210 us).
static int atc_parts(int max_tiles, int num_kv_heads, int max_context, long long scratch_floats) {
  const long long units = (long long)max_tiles * num_kv_heads;
  const int sms = atc_num_sms();
  const int key_tiles = (max_context + ATC_KEYS - 1) / ATC_KEYS;
  if (units <= 0 || 4 * units > 5ll * sms) return 1;
  if (units > sms)  // a few multiprocessors hold two blocks and set the time: two parts, for long chains only
    return key_tiles >= ATC_TWO_WAVE_TILES && units * 2 * ATC_PART_FLOATS <= scratch_floats ? 2 : 1;
  int parts = (int)(2ll * sms / units);
  if (parts > key_tiles / ATC_MIN_PART_TILES) parts = key_tiles / ATC_MIN_PART_TILES;
  if (parts > ATC_MAX_PARTS) parts = ATC_MAX_PARTS;
  if (parts < 2 || units * parts * ATC_PART_FLOATS > scratch_floats) return 1;
  const float whole = key_tiles * 1.3f + 6.0f;
  const float cut = (float)key_tiles / parts * (units * parts <= sms ? 1.3f : 1.9f) + 12.0f;
  return cut < 0.85f * whole ? parts : 1;
}

TS_EXPORT int ts_flash_prefill_tc_parts(int max_tiles, int num_kv_heads, int max_context, long long scratch_floats) {
  return atc_parts(max_tiles, num_kv_heads, max_context, scratch_floats);
}

// Steps with prompts in them, head size 128.  max_tiles: an upper bound of the sum over requests
// of ceil(query_len / tokens_per_tile), tokens_per_tile = 128 / (num_heads / num_kv_heads).
TS_EXPORT int ts_flash_prefill_tc(const void* q, long long q_stride, void* out, long long out_stride,
                                  const void* k_pages, const void* v_pages, long long num_pages,
                                  const int* block_table, int table_stride, const int* query_start_loc,
                                  const int* context_lens, int num_seqs, int max_tiles, int page_size,
                                  int num_heads, int num_kv_heads, int head_dim, int window, float scale,
                                  float* part_scratch, long long scratch_floats, int max_context, int* status,
                                  cudaStream_t stream) {
  if (num_seqs <= 0 || max_tiles <= 0) return 0;
  if (head_dim != ATC_D) return TS_ERR_SIZE;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads) return TS_ERR_SIZE;
  if (num_heads / num_kv_heads > ATC_ROWS || (long long)max_tiles * num_kv_heads >= (1ll << 31) - 1) return TS_ERR_SIZE;
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  if ((1 << shift) != page_size || page_size < 4) return TS_ERR_SIZE;  // one producer lane per page of a tile
  if (((uintptr_t)q & 15) || ((uintptr_t)out & 15) || (q_stride & 7) || (out_stride & 7)) return TS_ERR_ALIGN;
  if (((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15)) return TS_ERR_ALIGN;
  if (!(scale > 0.0f)) return TS_ERR_ARGUMENT;
  const long long rows = num_pages * page_size;
  if (rows <= 0 || rows >= (1ll << 31) - 256) return TS_ERR_SIZE;
  const int box_rows = page_size < ATC_KEYS ? page_size : ATC_KEYS;
  CUtensorMap map_k, map_v;
  int code = atc_make_map(&map_k, k_pages, rows, (long long)num_kv_heads * head_dim, box_rows);
  if (code) return code;
  code = atc_make_map(&map_v, v_pages, rows, (long long)num_kv_heads * head_dim, box_rows);
  if (code) return code;
  const long long units = (long long)max_tiles * num_kv_heads;
  const int parts = atc_parts(max_tiles, num_kv_heads, max_context, part_scratch != nullptr ? scratch_floats : 0);
  const float scale_log2 = scale * 1.4426950408889634f;
  if (parts == 1) {
    cudaFuncSetAttribute(flash_prefill_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_SMEM);
    ts_launch(flash_prefill_tc_kernel<false>, dim3((unsigned)units), dim3(ATC_THREADS), ATC_SMEM, stream, map_k, map_v,
              (const bf16*)q, q_stride, (bf16*)out, out_stride, block_table, table_stride, query_start_loc,
              context_lens, num_seqs, shift, box_rows, (int)rows, num_heads, num_kv_heads, window, scale_log2, 1,
              (float*)nullptr, status);
    return ts_launch_status();
  }
  cudaFuncSetAttribute(flash_prefill_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_SMEM);
  ts_launch(flash_prefill_tc_kernel<true>, dim3((unsigned)(units * parts)), dim3(ATC_THREADS), ATC_SMEM, stream, map_k, map_v,
            (const bf16*)q, q_stride, (bf16*)out, out_stride, block_table, table_stride, query_start_loc,
            context_lens, num_seqs, shift, box_rows, (int)rows, num_heads, num_kv_heads, window, scale_log2, parts,
            part_scratch, status);
  code = ts_launch_status();
  if (code) return code;
  ts_launch(flash_prefill_tc_merge_kernel, dim3((unsigned)units), dim3(2 * ATC_ROWS), 0, stream, (const float*)part_scratch,
            parts, (bf16*)out, out_stride, query_start_loc, num_seqs, num_heads, num_kv_heads, scale_log2);
  return ts_launch_status();
}
