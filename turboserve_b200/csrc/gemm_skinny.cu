// C[M,N] = A[M,K] * W[N,K]^T (+ bias) for few rows (M <= 64), bfloat16 in, fp32 accumulate:
// the matrix product of decode steps, where every weight is read once and the time is the
// time to stream W from HBM.
//
// The weights sit on the 16-wide M side of mma.sync.m16n8k16 and the batch on its 8-wide N
// side.  A warp owns 16 weight rows over a slice of K and reads them straight from global
// memory into the fragment registers with 16-byte loads: within a 32-wide K chunk the thread
// (g, t) of the warp (g = lane / 4, t = lane % 4) loads elements 8t..8t+7 of rows g and g+8.
// The tensor-core fragment wants k-slots {2t, 2t+1, 2t+8, 2t+9} from that thread; since the
// same thread supplies the same slots of the activation fragment, any one-to-one assignment
// of physical k to slots gives the same dot product, so elements 8t..8t+3 feed one mma and
// 8t+4..8t+7 the next, with the activations loaded by the same rule.  Eight chunks are loaded
// before the first is used, which keeps enough bytes in flight to cover HBM latency.
//
// A block is 8 warps arranged as (8 / ksplit) row tiles x ksplit K slices; the K slices of a
// row tile are summed in shared memory in slice order (no atomics, no global scratch), then
// bias is added and the result stored as bf16 or fp32.  K must be a multiple of 8 and rows of
// A and W 16-byte aligned; any M <= 64 and any N.
//
// It stands where the reference calls F.linear on a decode batch
// (src/turboserve/engine/model/layers.py:142, src/turboserve/engine/model/model.py:243-244).
#include "common.cuh"

#define SKINNY_WARPS 8
#define UNROLL 8

__device__ __forceinline__ uint4 load16(const __nv_bfloat16* p, bool valid) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (valid) {
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
  }
  return v;
}

__device__ __forceinline__ uint4 load16_cached(const __nv_bfloat16* p, bool valid) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (valid) v = __ldg(reinterpret_cast<const uint4*>(p));
  return v;
}

__device__ __forceinline__ void mma_bf16(float (&d)[4], unsigned a0, unsigned a1, unsigned a2,
                                         unsigned a3, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// MT: number of 8-row batch tiles (M <= 8 * MT).  KSPLIT: K slices per row tile.
template <int MT, int KSPLIT, typename TOut>
__global__ void __launch_bounds__(SKINNY_WARPS * 32)
gemm_skinny_kernel(const __nv_bfloat16* __restrict__ a, long long lda,
                   const __nv_bfloat16* __restrict__ w, long long ldw,
                   const float* __restrict__ bias, TOut* __restrict__ c, long long ldc, int m,
                   int n, int k, int early_trigger) {
  constexpr int ROW_TILES = SKINNY_WARPS / KSPLIT;
  __shared__ float partial[KSPLIT > 1 ? SKINNY_WARPS : 1][MT * 4 * 32];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row_tile = warp / KSPLIT, slice = warp % KSPLIT;
  const int n0 = (blockIdx.x * ROW_TILES + row_tile) * 16;

  const int chunks = (k + 31) / 32;
  const int per_slice = (chunks + KSPLIT - 1) / KSPLIT;
  const int chunk_begin = slice * per_slice;
  const int chunk_end = min(chunks, chunk_begin + per_slice);

  const bool row_lo = n0 + g < n, row_hi = n0 + g + 8 < n;
  const __nv_bfloat16* w_lo = w + (size_t)(n0 + g) * ldw + 8 * t;
  const __nv_bfloat16* w_hi = w + (size_t)(n0 + g + 8) * ldw + 8 * t;

  float acc[MT][4];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // Two register buffers of U chunks each: the loads of the next U chunks are in flight while
  // the current U chunks feed the tensor cores.
  constexpr int U = MT <= 2 ? UNROLL : UNROLL / 2;
  auto issue = [&](uint4 (&lo)[U], uint4 (&hi)[U], int chunk) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kk = (chunk + u) * 32 + 8 * t;
      const bool in_k = (chunk + u) < chunk_end && kk < k;
      lo[u] = load16(w_lo + (size_t)(chunk + u) * 32, in_k && row_lo);
      hi[u] = load16(w_hi + (size_t)(chunk + u) * 32, in_k && row_hi);
    }
  };
  auto compute = [&](const uint4 (&lo)[U], const uint4 (&hi)[U], int chunk) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int kk = (chunk + u) * 32 + 8 * t;
      const bool in_k = (chunk + u) < chunk_end && kk < k;
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        const int row = mt * 8 + g;
        const uint4 x = load16_cached(a + (size_t)row * lda + kk, in_k && row < m);
        mma_bf16(acc[mt], lo[u].x, hi[u].x, lo[u].y, hi[u].y, x.x, x.y);
        mma_bf16(acc[mt], lo[u].z, hi[u].z, lo[u].w, hi[u].w, x.z, x.w);
      }
    }
  };
  uint4 lo0[U], hi0[U], lo1[U], hi1[U];
  issue(lo0, hi0, chunk_begin);  // weights: nothing before this kernel writes them
  pdl_wait();                    // activations come from the kernel before
  if (early_trigger) pdl_trigger<2>();  // not when the kernel after this one is launched as clusters (slow to launch early)
  for (int chunk = chunk_begin; chunk < chunk_end; chunk += 2 * U) {
    issue(lo1, hi1, chunk + U);
    compute(lo0, hi0, chunk);
    issue(lo0, hi0, chunk + 2 * U);
    compute(lo1, hi1, chunk + U);
  }

  if (KSPLIT > 1) {
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < 4; ++j) partial[warp][(mt * 4 + j) * 32 + lane] = acc[mt][j];
    __syncthreads();
    if (slice != 0) return;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float v = acc[mt][j];
        for (int s = 1; s < KSPLIT; ++s) v += partial[warp + s][(mt * 4 + j) * 32 + lane];
        acc[mt][j] = v;
      }
  }

  // acc[mt][0,1]: weight row n0+g,   batch rows mt*8 + 2t, 2t+1
  // acc[mt][2,3]: weight row n0+g+8, batch rows mt*8 + 2t, 2t+1
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = n0 + g + (j >= 2 ? 8 : 0);
      const int row = mt * 8 + 2 * t + (j & 1);
      if (col < n && row < m) {
        float v = acc[mt][j];
        if (bias) v += bias[col];
        c[(size_t)row * ldc + col] = from_float<TOut>(v);
      }
    }
  }
}

template <int MT, typename TOut>
static int launch_skinny(const __nv_bfloat16* a, long long lda, const __nv_bfloat16* w,
                         long long ldw, const float* bias, TOut* c, long long ldc, int m, int n,
                         int k, int ksplit, int early_trigger, cudaStream_t stream) {
  const int rows_per_block = 16 * SKINNY_WARPS / ksplit;
  const int grid = (n + rows_per_block - 1) / rows_per_block;
  switch (ksplit) {
    case 1: ts_launch(gemm_skinny_kernel<MT, 1, TOut>, dim3(grid), dim3(SKINNY_WARPS * 32), 0, stream, a, lda, w, ldw, bias, c, ldc, m, n, k, early_trigger); break;
    case 2: ts_launch(gemm_skinny_kernel<MT, 2, TOut>, dim3(grid), dim3(SKINNY_WARPS * 32), 0, stream, a, lda, w, ldw, bias, c, ldc, m, n, k, early_trigger); break;
    case 4: ts_launch(gemm_skinny_kernel<MT, 4, TOut>, dim3(grid), dim3(SKINNY_WARPS * 32), 0, stream, a, lda, w, ldw, bias, c, ldc, m, n, k, early_trigger); break;
    case 8: ts_launch(gemm_skinny_kernel<MT, 8, TOut>, dim3(grid), dim3(SKINNY_WARPS * 32), 0, stream, a, lda, w, ldw, bias, c, ldc, m, n, k, early_trigger); break;
    default: return TS_ERR_ARGUMENT;
  }
  return ts_launch_status();
}

template <typename TOut>
static int dispatch_skinny(const __nv_bfloat16* a, long long lda, const __nv_bfloat16* w,
                           long long ldw, const float* bias, TOut* c, long long ldc, int m, int n,
                           int k, int ksplit, int early_trigger, cudaStream_t stream) {
  if (m <= 8) return launch_skinny<1, TOut>(a, lda, w, ldw, bias, c, ldc, m, n, k, ksplit, early_trigger, stream);
  if (m <= 16) return launch_skinny<2, TOut>(a, lda, w, ldw, bias, c, ldc, m, n, k, ksplit, early_trigger, stream);
  if (m <= 32) return launch_skinny<4, TOut>(a, lda, w, ldw, bias, c, ldc, m, n, k, ksplit, early_trigger, stream);
  return launch_skinny<8, TOut>(a, lda, w, ldw, bias, c, ldc, m, n, k, ksplit, early_trigger, stream);
}

// early_trigger: whether the kernel lets the one after it in the stream be set up as soon as it
// has its own inputs (programmatic dependent launch); 0 holds the next kernel back until this one ends.
// ksplit: 0 lets the entry point choose (the smallest of 1, 2, 4, 8 that gives every SM two
// blocks, given the number of SMs of the current device); otherwise one of 1, 2, 4, 8.
TS_EXPORT int ts_gemm_skinny(int out_dtype, const void* a, long long lda, const void* w,
                             long long ldw, const float* bias, void* c, long long ldc, int m,
                             int n, int k, int ksplit, int num_sms, int early_trigger, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (m > 64) return TS_ERR_SIZE;
  if (k < 8 || k % 8) return TS_ERR_SIZE;
  if (lda % 8 || ldw % 8) return TS_ERR_ALIGN;
  if (((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return TS_ERR_ALIGN;
  if (ksplit == 0) {
    const int want = 2 * (num_sms > 0 ? num_sms : 148);
    ksplit = 8;
    for (int s = 1; s <= 8; s *= 2) {
      const int rows_per_block = 16 * SKINNY_WARPS / s;
      if ((n + rows_per_block - 1) / rows_per_block >= want) { ksplit = s; break; }
    }
    while (ksplit > 1 && (k + 31) / 32 < ksplit) ksplit /= 2;
  }
  const __nv_bfloat16* ap = (const __nv_bfloat16*)a;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
  if (out_dtype == TS_BF16)
    return dispatch_skinny<__nv_bfloat16>(ap, lda, wp, ldw, bias, (__nv_bfloat16*)c, ldc, m, n, k, ksplit, early_trigger, stream);
  if (out_dtype == TS_F32)
    return dispatch_skinny<float>(ap, lda, wp, ldw, bias, (float*)c, ldc, m, n, k, ksplit, early_trigger, stream);
  return TS_ERR_DTYPE;
}
