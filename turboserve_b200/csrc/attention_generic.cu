// Paged attention for any dtype, head size and head grouping: the 32-bit path of the model
// and the fallback for sizes the tensor-core kernels refuse.
//
// One block per (query token, query head).  The query at absolute position p sees keys lo..p
// of its own sequence, lo = max(0, p - window + 1) (window == 0: lo = 0), read from the paged
// cache through the sequence's block table; the keys of this step have been appended before
// the kernel runs, so a token sees itself.  Keys are taken in tiles of 32 counted from lo and
// dealt to GENERIC_STREAMS = 16 streams: stream s takes tiles s, s + 16, ...; one lane scores
// one key, then the tile's values are accumulated with every lane owning head dims lane,
// lane + 32, ...  The sixteen partial results are merged in stream order.  The order of every
// sum is therefore a function of (lo, p) alone: the output of a token does not depend on how
// the sequence was cut into steps or on what else is in the batch.  How many warps work the
// streams does not change a bit either: a step of many tokens runs four warps a block, each
// four streams one after the other; a step of few tokens (decoding) sixteen warps, one each.
//
// Scores, softmax (natural exp, running maximum) and the value sum are fp32; the output is
// rounded once.  What it replaces in the reference: gather + mask + SDPA per sequence
// (src/turboserve/engine/model/attention.py:139-148,184-209) with scale = head_dim^-0.5
// (src/turboserve/engine/model/model_config.py:224-227).
#include "common.cuh"

#define GENERIC_STREAMS 16
#define MAX_DIMS_PER_LANE 8  // head_dim <= 256

// blockDim.x / 32 warps, a divisor of GENERIC_STREAMS
template <typename T>
__global__ void __launch_bounds__(GENERIC_STREAMS * 32)
paged_attention_generic_kernel(const T* __restrict__ q, long long q_stride, T* __restrict__ out,
                               long long out_stride, const T* __restrict__ k_pages,
                               const T* __restrict__ v_pages, const int* __restrict__ block_table,
                               int table_stride, const int* __restrict__ seq_of_token,
                               const int* __restrict__ positions, int page_size, int num_heads,
                               int num_kv_heads, int head_dim, int window, float scale,
                               int* __restrict__ status) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float smem[];
  float* q_s = smem;                               // [head_dim]
  float* part_acc = smem + head_dim;               // [GENERIC_STREAMS][head_dim]
  float* part_ml = part_acc + GENERIC_STREAMS * head_dim;  // [GENERIC_STREAMS][2]

  const int t = blockIdx.x, head = blockIdx.y;
  const int seq = seq_of_token[t];
  if (seq < 0) return;
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int kv_head = head / (num_heads / num_kv_heads);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, num_warps = blockDim.x >> 5;
  const int* table = block_table + (size_t)seq * table_stride;

  const T* q_row = q + (size_t)t * q_stride + (size_t)head * head_dim;
  for (int i = threadIdx.x; i < head_dim; i += blockDim.x) q_s[i] = to_float(q_row[i]);
  __syncthreads();

  const int num_keys = pos - lo + 1;
  const int num_tiles = (num_keys + 31) / 32;
  const bool wide = sizeof(T) == 4 && head_dim % 4 == 0 && !((uintptr_t)k_pages & 15);  // key rows are 16-byte aligned
  for (int stream = warp; stream < GENERIC_STREAMS; stream += num_warps) {
    float m = -INFINITY, l = 0.0f;
    float acc[MAX_DIMS_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) acc[i] = 0.0f;
    for (int tile = stream; tile < num_tiles; tile += GENERIC_STREAMS) {
      const int key = lo + tile * 32 + lane;
      const bool valid = key <= pos;
      float s = -INFINITY;
      size_t row = 0;
      if (valid) {
        const int page = table[key / page_size];
        if (page < 0) {
          if (status) atomicOr(status, 4);
        } else {
          row = (((size_t)page * page_size + key % page_size) * num_kv_heads + kv_head) * head_dim;
          const T* k_row = k_pages + row;
          float dot = 0.0f;
          if (wide) {  // the same products in the same order, four to a load
            const float4* k4 = reinterpret_cast<const float4*>(k_row);
            for (int i = 0; i < head_dim / 4; ++i) {
              const float4 kv = k4[i];
              dot = fmaf(q_s[4 * i], kv.x, dot);
              dot = fmaf(q_s[4 * i + 1], kv.y, dot);
              dot = fmaf(q_s[4 * i + 2], kv.z, dot);
              dot = fmaf(q_s[4 * i + 3], kv.w, dot);
            }
          } else {
            for (int i = 0; i < head_dim; ++i) dot = fmaf(q_s[i], to_float(k_row[i]), dot);
          }
          s = dot * scale;
        }
      }
      const float tile_max = warp_max(s);
      const float m_new = fmaxf(m, tile_max);
      if (m_new == -INFINITY) continue;  // only unreadable keys so far
      const float corr = expf(m - m_new);
      const float p = s == -INFINITY ? 0.0f : expf(s - m_new);
      l = l * corr + warp_sum(p);
#pragma unroll
      for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) acc[i] *= corr;
      m = m_new;
      const int in_tile = min(32, pos - (lo + tile * 32) + 1);
      for (int j = 0; j < in_tile; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const unsigned long long rj = __shfl_sync(0xffffffffu, (unsigned long long)row, j);
        if (pj == 0.0f) continue;
        const T* v_row = v_pages + rj;
#pragma unroll
        for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
          const int dim = lane + 32 * i;
          if (dim < head_dim) acc[i] = fmaf(pj, to_float(v_row[dim]), acc[i]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < MAX_DIMS_PER_LANE; ++i) {
      const int dim = lane + 32 * i;
      if (dim < head_dim) part_acc[stream * head_dim + dim] = acc[i];
    }
    if (lane == 0) {
      part_ml[stream * 2] = m;
      part_ml[stream * 2 + 1] = l;
    }
  }
  __syncthreads();
  if (warp == 0) {
    float m_all = -INFINITY;
    for (int w = 0; w < GENERIC_STREAMS; ++w) m_all = fmaxf(m_all, part_ml[w * 2]);
    float weight[GENERIC_STREAMS];
    float l_all = 0.0f;
    for (int w = 0; w < GENERIC_STREAMS; ++w) {
      const float mw = part_ml[w * 2];
      weight[w] = mw == -INFINITY ? 0.0f : expf(mw - m_all);
      l_all += part_ml[w * 2 + 1] * weight[w];
    }
    const float inv = l_all > 0.0f ? 1.0f / l_all : 0.0f;
    T* o_row = out + (size_t)t * out_stride + (size_t)head * head_dim;
    for (int dim = lane; dim < head_dim; dim += 32) {
      float v = 0.0f;
      for (int w = 0; w < GENERIC_STREAMS; ++w) v += part_acc[w * head_dim + dim] * weight[w];
      o_row[dim] = from_float<T>(v * inv);
    }
  }
}

TS_EXPORT int ts_paged_attention_generic(int dtype, const void* q, long long q_stride, void* out,
                                         long long out_stride, const void* k_pages,
                                         const void* v_pages, const int* block_table,
                                         int table_stride, const int* seq_of_token,
                                         const int* positions, int num_tokens, int page_size,
                                         int num_heads, int num_kv_heads, int head_dim, int window,
                                         float scale, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (head_dim < 1 || head_dim > 32 * MAX_DIMS_PER_LANE) return TS_ERR_SIZE;
  if (num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads) return TS_ERR_SIZE;
  if (num_heads > 65535 || page_size < 1 || window < 0) return TS_ERR_ARGUMENT;
  dim3 grid(num_tokens, num_heads);
  const size_t smem = ((size_t)head_dim * (1 + GENERIC_STREAMS) + 2 * GENERIC_STREAMS) * sizeof(float);
  // few blocks (a decode step): a warp per stream; many: four warps, four streams each
  const int threads = (long long)num_tokens * num_heads <= 2048 ? GENERIC_STREAMS * 32 : 4 * 32;
  if (dtype == TS_F32)
    ts_launch(paged_attention_generic_kernel<float>, dim3(grid), dim3(threads), smem, stream, 
        (const float*)q, q_stride, (float*)out, out_stride, (const float*)k_pages,
        (const float*)v_pages, block_table, table_stride, seq_of_token, positions, page_size,
        num_heads, num_kv_heads, head_dim, window, scale, status);
  else if (dtype == TS_BF16)
    ts_launch(paged_attention_generic_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), smem, stream, 
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride,
        (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, block_table, table_stride,
        seq_of_token, positions, page_size, num_heads, num_kv_heads, head_dim, window, scale,
        status);
  else
    return TS_ERR_DTYPE;
  return ts_launch_status();
}
