// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) on the CUDA cores with fp32 FFMA: the matrix
// product of the true 32-bit path (no TF32, no tensor cores), also taken by bf16 shapes
// that the tensor-core kernels refuse.  Any M, N, K.
//
// Three forms of one sum.  Up to 16 rows of float32 (decode steps on the float32 path): a
// weight-streaming kernel, one warp per 32 output features, which reads every weight once at
// a good share of the memory bandwidth (below).  Up to 64 rows: a 64x64 output tile per block, 16-wide K steps
// staged in shared memory, a 4x4 micro-tile per thread.  More rows (prompts on the float32
// path): a 128x128 tile, an 8x8 micro-tile per thread, the next K step fetched into registers
// (16 bytes at a time where rows are aligned) while the current one is multiplied, two buffers
// of shared memory.  In both every output element accumulates its K products in increasing k,
// one FFMA each, so a row's result does not depend on M, on the tiling or on which tile the row
// falls into: all three give the same bits.
// It stands where the reference calls F.linear (src/turboserve/engine/model/layers.py:142).
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TIn* __restrict__ a, long long lda, const TIn* __restrict__ w,
                 long long ldw, const float* __restrict__ bias, TOut* __restrict__ c,
                 long long ldc, int m, int n, int k) {
  pdl_wait();
  pdl_trigger();
  __shared__ float a_s[BK][BM + 4];
  __shared__ float w_s[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tile_m = blockIdx.y * BM, tile_n = blockIdx.x * BN;
  const int tx = tid % 16, ty = tid / 16;  // tx -> columns (n), ty -> rows (m)
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  const int load_row = tid / 4;        // 0..63
  const int load_col = (tid % 4) * 4;  // 0,4,8,12
  for (int k0 = 0; k0 < k; k0 += BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int kk = k0 + load_col + e;
      const int am = tile_m + load_row, wn = tile_n + load_row;
      a_s[load_col + e][load_row] = (am < m && kk < k) ? to_float(a[(size_t)am * lda + kk]) : 0.0f;
      w_s[load_col + e][load_row] = (wn < n && kk < k) ? to_float(w[(size_t)wn * ldw + kk]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = a_s[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = w_s[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = tile_m + ty * 4 + i;
    if (row >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = tile_n + tx * 4 + j;
      if (col >= n) continue;
      float v = acc[i][j];
      if (bias) v += bias[col];
      c[(size_t)row * ldc + col] = from_float<TOut>(v);
    }
  }
}

// The 128x128 tiling (see the head of the file).  256 threads: thread (ty, tx) owns rows
// ty * 8 .. + 7 and columns tx * 4 .. + 3 and 64 + tx * 4 .. + 3 of the tile (two runs of four, so
// that a warp's reads of the weights' tile fall into different banks).
#define LM 128
#define LN 128
#define LK 16
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_simt_large_kernel(const TIn* __restrict__ a, long long lda, const TIn* __restrict__ w,
                       long long ldw, const float* __restrict__ bias, TOut* __restrict__ c,
                       long long ldc, int m, int n, int k, int vector_ok) {
  pdl_wait();
  pdl_trigger();
  __shared__ __align__(16) float a_s[2][LK][LM + 4];
  __shared__ __align__(16) float w_s[2][LK][LN + 4];
  const int tid = threadIdx.x;
  const int tile_m = blockIdx.y * LM, tile_n = blockIdx.x * LN;
  const int tx = tid % 16, ty = tid / 16;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

  // a tile is 128 rows x 16 k: thread t fetches k 4 * (t % 4) .. + 3 of rows t / 4 and 64 + t / 4
  const int load_row = tid / 4, load_k = (tid % 4) * 4;
  float ra[2][4], rw[2][4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int am = tile_m + load_row + 64 * h, wn = tile_n + load_row + 64 * h;
      const int kk = k0 + load_k;
      if (vector_ok && kk + 3 < k) {
        float4 va = make_float4(0.0f, 0.0f, 0.0f, 0.0f), vw = va;
        if (am < m) va = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a) + (size_t)am * lda + kk);
        if (wn < n) vw = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(w) + (size_t)wn * ldw + kk);
        ra[h][0] = va.x; ra[h][1] = va.y; ra[h][2] = va.z; ra[h][3] = va.w;
        rw[h][0] = vw.x; rw[h][1] = vw.y; rw[h][2] = vw.z; rw[h][3] = vw.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          ra[h][e] = (am < m && kk + e < k) ? to_float(a[(size_t)am * lda + kk + e]) : 0.0f;
          rw[h][e] = (wn < n && kk + e < k) ? to_float(w[(size_t)wn * ldw + kk + e]) : 0.0f;
        }
      }
    }
  };
  auto stage = [&](int buf) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        a_s[buf][load_k + e][load_row + 64 * h] = ra[h][e];
        w_s[buf][load_k + e][load_row + 64 * h] = rw[h][e];
      }
  };
  fetch(0);
  stage(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < k; k0 += LK) {
    const bool more = k0 + LK < k;
    if (more) fetch(k0 + LK);  // in flight while this step is multiplied
#pragma unroll
    for (int kk = 0; kk < LK; ++kk) {
      const float4 a0 = *reinterpret_cast<const float4*>(&a_s[buf][kk][ty * 8]);
      const float4 a1 = *reinterpret_cast<const float4*>(&a_s[buf][kk][ty * 8 + 4]);
      const float4 w0 = *reinterpret_cast<const float4*>(&w_s[buf][kk][tx * 4]);
      const float4 w1 = *reinterpret_cast<const float4*>(&w_s[buf][kk][64 + tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    if (more) {
      stage(buf ^ 1);  // the other buffer: nobody reads it during this step
      __syncthreads();
      buf ^= 1;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int row = tile_m + ty * 8 + i;
    if (row >= m) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int col = tile_n + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
      if (col >= n) continue;
      float v = acc[i][j];
      if (bias) v += bias[col];
      c[(size_t)row * ldc + col] = from_float<TOut>(v);
    }
  }
}

// The weight-streaming form for at most 16 rows of float32.  A block of four warps owns 32
// output features; lane f of every warp owns feature f, and each warp a quarter of the ROWS
// rows.  The block brings tiles of 32 features x 64 k of the weights (and ROWS x 64 k of the
// activations) into a ring of shared-memory stages with 16-byte cp.async (sixteen consecutive
// threads fetch 256 consecutive bytes of one weight row; what lies beyond n, m or k is filled
// with zeros, which leave a sum as it is), and every lane walks its row of a stage in
// increasing k, four k at a time.  Few features (less than four blocks a multiprocessor) get a
// deeper ring, so that a lone block still keeps about 50 KB on its way.
// Measured on B200 at 8 rows (weights of a 7B layer from HBM): 3.4 TB/s on the gate+up
// projection (1,184 blocks), 1.7 to 2.1 TB/s on the three with 3,584 or 4,608 features (112 and
// 144 blocks for 148 multiprocessors); the 64x64 tiling ran them at 0.2 to 0.85 TB/s.  What bounds
// it is shared memory: the activations reach the lanes as broadcast 16-byte loads, three loads
// for eight FFMA per lane, and a multiprocessor serves one such load in four cycles.  Two warps
// a block with four rows each, a 128-k stage, and operands fetched into registers one step
// ahead were all measured slower.
#define RN 32
#define RK 64
#define RPAD 4
#define RWARPS 4
template <int ROWS, int STAGES, typename TOut>
__global__ void __launch_bounds__(32 * RWARPS)
gemm_simt_rows_kernel(const float* __restrict__ a, long long lda, const float* __restrict__ w, long long ldw,
                      const float* __restrict__ bias, TOut* __restrict__ c, long long ldc, int m, int n, int k) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(16) float rows_smem[];
  constexpr int W_STAGE = RN * (RK + RPAD), A_STAGE = ROWS * (RK + RPAD), STAGE = W_STAGE + A_STAGE;
  constexpr int MINE = ROWS / RWARPS;  // rows a warp adds up
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n0 = blockIdx.x * RN;
  constexpr int CHUNKS = RK / 4, PER_PASS = 32 * RWARPS / CHUNKS;  // 16-byte chunks of a row's k in a stage; rows per pass
  const int chunk = threadIdx.x % CHUNKS, sub = threadIdx.x / CHUNKS;
  const int num_steps = (k + RK - 1) / RK;

  auto issue = [&](int step) {
    float* stage = rows_smem + (step % STAGES) * STAGE;
    const int kk = step * RK + chunk * 4;
    const int k_left = k - kk;  // floats of this chunk that exist
    const unsigned bytes_k = k_left >= 4 ? 16u : (k_left > 0 ? (unsigned)k_left * 4u : 0u);
#pragma unroll
    for (int pass = 0; pass < RN / PER_PASS; ++pass) {
      const int f = pass * PER_PASS + sub;
      const unsigned bytes = n0 + f < n ? bytes_k : 0u;
      const float* src = w + (size_t)(bytes ? n0 + f : 0) * ldw + (bytes ? kk : 0);
      const unsigned dst = (unsigned)__cvta_generic_to_shared(stage + f * (RK + RPAD) + chunk * 4);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    }
#pragma unroll
    for (int pass = 0; pass < (ROWS + PER_PASS - 1) / PER_PASS; ++pass) {
      const int r = pass * PER_PASS + sub;
      if (r >= ROWS) break;
      const unsigned bytes = r < m ? bytes_k : 0u;
      const float* src = a + (size_t)(bytes ? r : 0) * lda + (bytes ? kk : 0);
      const unsigned dst = (unsigned)__cvta_generic_to_shared(stage + W_STAGE + r * (RK + RPAD) + chunk * 4);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
    }
  };

  float acc[MINE];
#pragma unroll
  for (int r = 0; r < MINE; ++r) acc[r] = 0.0f;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < num_steps) issue(s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int step = 0; step < num_steps; ++step) {
    asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();  // every thread's copies of this stage have landed; everyone is done with the stage refilled next
    if (step + STAGES - 1 < num_steps) issue(step + STAGES - 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const float* stage = rows_smem + (step % STAGES) * STAGE;
    const float* w_row = stage + lane * (RK + RPAD);
    const float* a_rows = stage + W_STAGE + warp * MINE * (RK + RPAD);
#pragma unroll
    for (int kk = 0; kk < RK; kk += 4) {
      const float4 wv = *reinterpret_cast<const float4*>(w_row + kk);
#pragma unroll
      for (int r = 0; r < MINE; ++r) {
        const float4 av = *reinterpret_cast<const float4*>(a_rows + r * (RK + RPAD) + kk);
        acc[r] = fmaf(av.x, wv.x, acc[r]);
        acc[r] = fmaf(av.y, wv.y, acc[r]);
        acc[r] = fmaf(av.z, wv.z, acc[r]);
        acc[r] = fmaf(av.w, wv.w, acc[r]);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  const int col = n0 + lane;
  if (col >= n) return;
  const float b = bias ? bias[col] : 0.0f;
#pragma unroll
  for (int r = 0; r < MINE; ++r) {
    const int row = warp * MINE + r;
    if (row >= m) break;
    float v = acc[r];
    if (bias) v += b;
    c[(size_t)row * ldc + col] = from_float<TOut>(v);
  }
}

template <int ROWS, int STAGES>
static void launch_rows(const float* a, long long lda, const float* w, long long ldw, const float* bias, float* c,
                        long long ldc, int m, int n, int k, cudaStream_t stream) {
  const size_t smem = (size_t)STAGES * (RN + ROWS) * (RK + RPAD) * sizeof(float);
  cudaFuncSetAttribute(gemm_simt_rows_kernel<ROWS, STAGES, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  ts_launch(gemm_simt_rows_kernel<ROWS, STAGES, float>, dim3((n + RN - 1) / RN), dim3(32 * RWARPS), smem, stream, a, lda, w,
            ldw, bias, c, ldc, m, n, k);
}

static int simt_num_sms() {
  static int count = 0;
  if (count == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    if (count <= 0) count = 148;
  }
  return count;
}

template <typename TIn, typename TOut>
static void launch_simt(const void* a, long long lda, const void* w, long long ldw, const float* bias, void* c,
                        long long ldc, int m, int n, int k, cudaStream_t stream) {
  if constexpr (sizeof(TIn) == 4 && sizeof(TOut) == 4) {
    // rows of 16-byte aligned float32, at most 16 of them: the weight-streaming form
    if (m <= 16 && k > 0 && lda % 4 == 0 && ldw % 4 == 0 && !(((uintptr_t)a | (uintptr_t)w) & 15)) {
      const bool deep = (n + RN - 1) / RN < 4 * simt_num_sms();
      const float* af = (const float*)a;
      const float* wf = (const float*)w;
      if (m <= 8) {
        if (deep) launch_rows<8, 6>(af, lda, wf, ldw, bias, (float*)c, ldc, m, n, k, stream);
        else launch_rows<8, 3>(af, lda, wf, ldw, bias, (float*)c, ldc, m, n, k, stream);
      } else {
        if (deep) launch_rows<16, 6>(af, lda, wf, ldw, bias, (float*)c, ldc, m, n, k, stream);
        else launch_rows<16, 3>(af, lda, wf, ldw, bias, (float*)c, ldc, m, n, k, stream);
      }
      return;
    }
  }
  if (m > BM) {
    const bool fp32 = sizeof(TIn) == 4;
    const int vector_ok = fp32 && lda % 4 == 0 && ldw % 4 == 0 && !(((uintptr_t)a | (uintptr_t)w) & 15);
    dim3 grid((n + LN - 1) / LN, (m + LM - 1) / LM);
    ts_launch(gemm_simt_large_kernel<TIn, TOut>, grid, dim3(256), 0, stream, (const TIn*)a, lda, (const TIn*)w, ldw,
              bias, (TOut*)c, ldc, m, n, k, vector_ok);
    return;
  }
  dim3 grid((n + BN - 1) / BN, (m + BM - 1) / BM);
  ts_launch(gemm_simt_kernel<TIn, TOut>, grid, dim3(256), 0, stream, (const TIn*)a, lda, (const TIn*)w, ldw, bias,
            (TOut*)c, ldc, m, n, k);
}

// out_dtype: dtype code of C (TS_F32 is allowed with bf16 inputs: logits).
TS_EXPORT int ts_gemm_simt(int dtype, int out_dtype, const void* a, long long lda, const void* w,
                           long long ldw, const float* bias, void* c, long long ldc, int m, int n,
                           int k, cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  if (k < 0) return TS_ERR_SIZE;
  if ((m + BM - 1) / BM > 65535) return TS_ERR_SIZE;
  if (dtype == TS_F32 && out_dtype == TS_F32)
    launch_simt<float, float>(a, lda, w, ldw, bias, c, ldc, m, n, k, stream);
  else if (dtype == TS_BF16 && out_dtype == TS_BF16)
    launch_simt<__nv_bfloat16, __nv_bfloat16>(a, lda, w, ldw, bias, c, ldc, m, n, k, stream);
  else if (dtype == TS_BF16 && out_dtype == TS_F32)
    launch_simt<__nv_bfloat16, float>(a, lda, w, ldw, bias, c, ldc, m, n, k, stream);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}
