// Sampling: one block per row of fp32 logits turns the row into one token id.
//
// Stages, in the reference's order (src/turboserve/engine/core/sampler.py:190-238):
//   repetition penalty (CTRL rule, :83-122)  ->  log-probabilities, if asked (:222-223)
//   -> temperature (:125-135) -> top-k (:138-148) -> top-p (:151-168) -> draw (:258-297).
// A row with temperature 0 is greedy: the argmax of the penalised logits, lowest id on ties.
// Other rows draw from softmax(row) with the Gumbel-max rule: argmax_i(x_i + g_i),
// g_i = -log(-log(u_i)), where u_i is a counter-based uniform that depends only on the
// request's seed, the index of the token being generated and the vocabulary id i.  A
// request's draws therefore do not depend on its neighbours in the batch.
//
// top-k keeps the values >= the k-th largest, found by a radix select over the ordered bits
// of the floats.  top-p keeps a token iff the probability mass of strictly larger values is
// <= p, found by the same radix descent over masses held in 2^-40 fixed point, so that the
// atomics that build the histograms are exact integer sums and the result is deterministic.
//
// `work` ([rows, vocab] fp32) is scratch owned by the caller; its contents are dead after
// the call.
//
// A row may be cut into `chunks` parts along the vocabulary, one block each (grid = rows x
// chunks), when all it needs is one pass: a greedy row, or a draw with neither top-k nor top-p
// (no penalty, no log-probability either).  Every part finds its own best (value, id), leaves
// it in `partial`, and the part that finishes last (an atomic count per row, no waiting) picks
// among them; "larger value, lower id on ties" does not depend on the order.  A row that wants
// its log-probability also leaves each part's maximum and sum of exponentials, which the last
// part adds up in the order of the parts.  A row that needs the filters is worked by its first
// block alone.  `partial` holds rows * (4 * chunks + 1) words and its counters must be zero
// before the first call; the kernel leaves them zero.
//
// Options may also be looked up by state slot (RowLookup, filled from a step's own index arrays):
// row -> the step's token whose logits it holds (row_token, or the row itself) -> that token's
// request in the step (seq_of_token, or the token itself; negative: padding, the row is skipped)
// -> the request's state slot (seq_slot) and its length after the step (seq_context).  The
// arrays temperature, top_k, top_p, penalty, want_logprob, seed and prompt_len are then indexed
// by the slot, and the index of the token being generated is seq_context - prompt_len[slot] (the
// request's length after the step minus its prompt), so nothing on the device has to be
// advanced from step to step.
//
// By slot, a request's history for the repetition penalty is a bitmap over the vocabulary
// (`seen`, seen_words 32-bit words per slot): bit t is set once token t is among the request's
// tokens.  ts_mark_seen sets the bits of the tokens a step runs (the portions of a prompt; after
// a preemption, of everything that is computed again), and a row sampled by slot first sets the
// bit of the token its logits come from (`step_tokens`, per token of the step: in a decode step
// the token sampled one step before), so the bitmap holds the whole sequence when the penalty reads it and nothing
// has to come from the host.  Whoever gives a slot to a new request clears its words first.
// Setting a bit twice changes nothing, so every block of a row may do it on its own.
#include "common.cuh"

#define SAMPLE_THREADS 1024
#define HIST_COPIES 16

__device__ __forceinline__ unsigned int ordered_key(float v) {
  const unsigned int bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__device__ __forceinline__ float key_to_float(unsigned int key) {
  const unsigned int bits = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
  return __uint_as_float(bits);
}

__host__ __device__ __forceinline__ float sample_uniform(unsigned long long seed,
                                                         unsigned int counter, unsigned int index) {
  unsigned long long x = (seed * 0x9E3779B97F4A7C15ull) ^
                         (((unsigned long long)counter << 32) | (unsigned long long)index);
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return ((float)(unsigned int)(x >> 41) + 0.5f) * (1.0f / 8388608.0f);  // 23 bits: exact, in (0, 1)
}

// The CTRL rule on one logit: a token that the request has seen becomes less likely whatever its sign.
// `seen_row` is null for a row without a penalty.
__device__ __forceinline__ float penalised(float v, int i, float pen, const unsigned int* seen_row) {
  if (seen_row != nullptr && ((__ldcg(&seen_row[i >> 5]) >> (i & 31)) & 1u)) v = v < 0.0f ? v * pen : v / pen;
  return v;
}

// How a row finds its request in the index arrays of a step (see the head of this file).
struct RowLookup {
  const int* row_token;     // per row, or null: token = row
  const int* seq_of_token;  // per token, or null: request = token
  const int* seq_slot;      // per request; null: options are per row, not by slot
  const int* seq_context;   // per request
  const int* step_tokens;   // per token, or null
};

struct ArgMax {
  float value;
  int index;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  if (b.value > a.value || (b.value == a.value && b.index < a.index)) return b;
  return a;
}

__device__ ArgMax block_argmax(ArgMax v, ArgMax* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    ArgMax o;
    o.value = __shfl_xor_sync(0xffffffffu, v.value, offset);
    o.index = __shfl_xor_sync(0xffffffffu, v.index, offset);
    v = better(v, o);
  }
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    ArgMax t = lane < (blockDim.x >> 5) ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      ArgMax o;
      o.value = __shfl_xor_sync(0xffffffffu, t.value, offset);
      o.index = __shfl_xor_sync(0xffffffffu, t.index, offset);
      t = better(t, o);
    }
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

#define FAST_BINS 4
// Sums of FAST_BINS + 1 64-bit integers over the block (exact, so the order is immaterial);
// every thread gets the totals.  scratch: 33 * (FAST_BINS + 1) words.
__device__ void block_sum_u64(unsigned long long (&v)[FAST_BINS + 1], unsigned long long* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int j = 0; j <= FAST_BINS; ++j)
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v[j] += __shfl_xor_sync(0xffffffffu, v[j], offset);
  __syncthreads();
  if (lane == 0)
#pragma unroll
    for (int j = 0; j <= FAST_BINS; ++j) scratch[warp * (FAST_BINS + 1) + j] = v[j];
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int j = 0; j <= FAST_BINS; ++j) {
      unsigned long long t = lane < (int)(blockDim.x >> 5) ? scratch[lane * (FAST_BINS + 1) + j] : 0ull;
#pragma unroll
      for (int offset = 16; offset > 0; offset >>= 1) t += __shfl_xor_sync(0xffffffffu, t, offset);
      if (lane == 0) scratch[32 * (FAST_BINS + 1) + j] = t;
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j <= FAST_BINS; ++j) v[j] = scratch[32 * (FAST_BINS + 1) + j];
  __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, long long logits_stride, float* __restrict__ work,
              int vocab, const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ penalty,
              const unsigned long long* __restrict__ seed, const unsigned int* __restrict__ counter,
              const int* __restrict__ history, const int* __restrict__ history_start,
              int* __restrict__ tokens, float* __restrict__ logprobs, const RowLookup look,
              const int* __restrict__ prompt_len, int* __restrict__ partial, int skip_filtered,
              const int* __restrict__ want_logprob, unsigned int* __restrict__ seen, int seen_words) {
  pdl_wait();
  pdl_trigger();
  __shared__ ArgMax arg_scratch[33];
  __shared__ float f_scratch[33];
  __shared__ unsigned long long hist64[256];
  __shared__ unsigned int hist32[256];
  // HIST_COPIES copies of a histogram, one per residue of the thread index: atomics on one
  // shared-memory word are served one after the other, and a row's values crowd into a few bins
  __shared__ unsigned long long hist_copies[HIST_COPIES * 256];
  unsigned int* const hist_copies32 = reinterpret_cast<unsigned int*>(hist_copies);
  const int copy = threadIdx.x & (HIST_COPIES - 1);
  __shared__ unsigned long long sum_scratch[33 * (FAST_BINS + 1)];
  __shared__ int sel_found;
  __shared__ unsigned int sel_prefix;
  __shared__ unsigned long long sel_above;
  __shared__ unsigned int sel_remaining;

  const int row = blockIdx.x;
  const bool by_slot = look.seq_slot != nullptr;
  int step_token = row, seq = row;
  if (by_slot) {
    step_token = look.row_token ? look.row_token[row] : row;
    seq = look.seq_of_token ? look.seq_of_token[step_token] : step_token;
    if (seq < 0) return;  // a padding row of a fixed-size batch
  }
  const int opt = by_slot ? look.seq_slot[seq] : row;  // where this row's options are
  const float* x = logits + (size_t)row * logits_stride;
  float* w = work + (size_t)row * vocab;
  const int tid = threadIdx.x;
  const float temp = temperature ? temperature[opt] : 0.0f;
  const float pen = penalty ? penalty[opt] : 1.0f;
  const bool need_lse = logprobs != nullptr && (want_logprob == nullptr || want_logprob[opt] != 0);
  // by slot the history is the slot's bitmap; the token this request ran in this step joins it first
  unsigned int* const seen_row = (by_slot && seen && pen != 1.0f) ? seen + (size_t)opt * seen_words : nullptr;
  if (seen_row != nullptr && look.step_tokens != nullptr) {
    const int t = look.step_tokens[step_token];
    if (tid == 0 && t >= 0 && t < vocab) atomicOr(&seen_row[t >> 5], 1u << (t & 31));
    __syncthreads();
  }
  const int k = top_k ? top_k[opt] : 0;
  const float p_option = top_p ? top_p[opt] : 1.0f;
  const unsigned long long sd = seed ? seed[opt] : 0ull;
  const unsigned int ctr = by_slot ? (unsigned int)(look.seq_context[seq] - prompt_len[opt]) : (counter ? counter[row] : 0u);

  // -- one pass is enough: greedy, or a draw without filters ----------------------------------
  const int chunks = gridDim.y;
  const bool one_pass = (pen == 1.0f || seen_row != nullptr) && (temp == 0.0f || (!(k > 0 && k < vocab) && !(p_option < 1.0f)));
  if (one_pass && partial != nullptr) {
    const int per = (vocab + chunks - 1) / chunks;
    const int lo = blockIdx.y * per, hi = min(vocab, lo + per);
    ArgMax pick{-INFINITY, 0x7fffffff};
    if (temp == 0.0f) {
      for (int i = lo + tid; i < hi; i += blockDim.x) pick = better(pick, ArgMax{penalised(x[i], i, pen, seen_row), i});
    } else {
      for (int i = lo + tid; i < hi; i += blockDim.x) {
        const float v = penalised(x[i], i, pen, seen_row) / temp;
        if (v == -INFINITY) continue;
        const float u = sample_uniform(sd, ctr, (unsigned int)i);
        pick = better(pick, ArgMax{v - logf(-logf(u)), i});
      }
    }
    pick = block_argmax(pick, arg_scratch);
    // for a log-probability: this part's maximum and its sum of exponentials of the penalised logits
    float part_max = -INFINITY, part_sum = 0.0f;
    if (need_lse) {
      for (int i = lo + tid; i < hi; i += blockDim.x) part_max = fmaxf(part_max, penalised(x[i], i, pen, seen_row));
      part_max = block_max(part_max, f_scratch);
      for (int i = lo + tid; i < hi; i += blockDim.x) part_sum += expf(penalised(x[i], i, pen, seen_row) - part_max);
      part_sum = block_sum(part_sum, f_scratch);
    }
    if (chunks == 1) {
      if (tid == 0) {
        tokens[row] = pick.index;
        if (need_lse) logprobs[row] = penalised(x[pick.index], pick.index, pen, seen_row) - (part_max + logf(part_sum));
      }
      return;
    }
    // per row: a counter, then (value, id) of every part, then (maximum, sum) of every part
    int* mine = partial + (size_t)row * (4 * chunks + 1);
    if (tid == 0) {
      mine[1 + 2 * blockIdx.y] = __float_as_int(pick.value);
      mine[2 + 2 * blockIdx.y] = pick.index;
      if (need_lse) {
        mine[1 + 2 * chunks + 2 * blockIdx.y] = __float_as_int(part_max);
        mine[2 + 2 * chunks + 2 * blockIdx.y] = __float_as_int(part_sum);
      }
      __threadfence();
      if (atomicAdd(&mine[0], 1) == chunks - 1) {  // every other part has left its results behind
        __threadfence();
        ArgMax all{-INFINITY, 0x7fffffff};
        for (int c = 0; c < chunks; ++c)
          all = better(all, ArgMax{__int_as_float(__ldcg(&mine[1 + 2 * c])), __ldcg(&mine[2 + 2 * c])});
        tokens[row] = all.index;
        if (need_lse) {  // the parts' sums brought to the row's maximum, added in the order of the parts
          float row_max = -INFINITY, row_sum = 0.0f;
          for (int c = 0; c < chunks; ++c) row_max = fmaxf(row_max, __int_as_float(__ldcg(&mine[1 + 2 * chunks + 2 * c])));
          for (int c = 0; c < chunks; ++c)
            row_sum += __int_as_float(__ldcg(&mine[2 + 2 * chunks + 2 * c])) * expf(__int_as_float(__ldcg(&mine[1 + 2 * chunks + 2 * c])) - row_max);
          logprobs[row] = penalised(x[all.index], all.index, pen, seen_row) - (row_max + logf(row_sum));
        }
        mine[0] = 0;
      }
    }
    return;
  }
  if (blockIdx.y != 0) return;  // a row that needs more than one pass is its first block's alone
  if (skip_filtered && by_slot && temp > 0.0f && ((k > 0 && k < vocab) || p_option < 1.0f)) return;  // the cluster kernel that follows draws it

  // -- repetition penalty ---------------------------------------------------------------
  for (int i = tid; i < vocab; i += blockDim.x) w[i] = penalised(x[i], i, pen, seen_row);
  if (pen != 1.0f && history_start) {
    __syncthreads();
    const int h0 = history_start[row], h1 = history_start[row + 1];
    for (int h = h0 + tid; h < h1; h += blockDim.x) {
      const int id = history[h];
      if (id >= 0 && id < vocab) {
        const float v = x[id];
        w[id] = v < 0.0f ? v * pen : v / pen;  // duplicates write the same value
      }
    }
  }
  __syncthreads();

  // -- greedy ---------------------------------------------------------------------------
  ArgMax best{-INFINITY, 0x7fffffff};
  if (temp == 0.0f || need_lse) {
    for (int i = tid; i < vocab; i += blockDim.x) best = better(best, ArgMax{w[i], i});
    best = block_argmax(best, arg_scratch);
  }
  float lse = 0.0f;
  if (need_lse) {
    float s = 0.0f;
    for (int i = tid; i < vocab; i += blockDim.x) s += expf(w[i] - best.value);
    lse = best.value + logf(block_sum(s, f_scratch));
  }
  if (temp == 0.0f) {
    if (tid == 0) {
      tokens[row] = best.index;
      if (need_lse) logprobs[row] = w[best.index] - lse;
    }
    return;
  }

  // -- temperature ------------------------------------------------------------------------
  // The value before scaling is needed for the log-probability of the drawn token, so the
  // scaled row goes back into `work` and the unscaled value is recomputed at the end.
  for (int i = tid; i < vocab; i += blockDim.x) w[i] = w[i] / temp;
  __syncthreads();

  // -- top-k ----------------------------------------------------------------------------------
  if (k > 0 && k < vocab) {
    if (tid == 0) { sel_prefix = 0; sel_remaining = (unsigned int)k; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < HIST_COPIES * 256; b += blockDim.x) hist_copies32[b] = 0;
      __syncthreads();
      const unsigned int prefix = sel_prefix;
      const unsigned int mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      // Values of one row crowd into a few bins (the leading byte is sign and exponent), and atomics
      // on one shared-memory word are served one after the other: a thread adds up what falls into
      // the same bin in a row and issues one atomic per run.  Integer sums: the order is immaterial.
      unsigned int run_bin = 256u, run_count = 0u;
      for (int i = tid; i < vocab; i += blockDim.x) {
        const unsigned int key = ordered_key(w[i]);
        if ((key & mask) != prefix) continue;
        const unsigned int bin = (key >> shift) & 255u;
        if (bin != run_bin) {
          if (run_count) atomicAdd(&hist_copies32[copy * 256 + run_bin], run_count);
          run_bin = bin;
          run_count = 0u;
        }
        ++run_count;
      }
      if (run_count) atomicAdd(&hist_copies32[copy * 256 + run_bin], run_count);
      __syncthreads();
      for (int b = tid; b < 256; b += blockDim.x) {
        unsigned int sum = 0u;
#pragma unroll
        for (int c = 0; c < HIST_COPIES; ++c) sum += hist_copies32[c * 256 + b];
        hist32[b] = sum;
      }
      __syncthreads();
      if (tid == 0) {
        unsigned int remaining = sel_remaining;
        int b = 255;
        for (; b > 0; --b) {
          if (hist32[b] >= remaining) break;
          remaining -= hist32[b];
        }
        sel_prefix = prefix | ((unsigned int)b << shift);
        sel_remaining = remaining;
      }
      __syncthreads();
    }
    const float threshold = key_to_float(sel_prefix);
    for (int i = tid; i < vocab; i += blockDim.x)
      if (w[i] < threshold) w[i] = -INFINITY;
    __syncthreads();
  }

  // -- top-p ----------------------------------------------------------------------------------
  const float p_keep = p_option;
  if (p_keep < 1.0f) {
    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += blockDim.x) mx = fmaxf(mx, w[i]);
    mx = block_max(mx, f_scratch);
    const float fixed_one = 1099511627776.0f;  // 2^40
    if (tid == 0) { sel_prefix = 0; sel_above = 0ull; sel_found = 0; }
    unsigned long long limit = 0ull;
    {
      // The first of the four radix passes sees every value of the row, and 64-bit atomics on
      // shared memory are slow (2.1 ms for this stage with them, 0.2 ms now).  The threshold nearly
      // always lies in one of the few highest bins that hold anything: their masses and the row's
      // total are kept in registers, added up over the block and walked as the histogram would be;
      // only if the threshold lies further down does the histogram pass run.  The sums are exact
      // integers either way, so the result is the same.  (For top-k, whose atomics are 32-bit, the
      // two extra scans of the row cost more than the pass they save.)
      const unsigned int top_bin = ordered_key(mx) >> 24;
      unsigned long long masses[FAST_BINS + 1] = {0ull, 0ull, 0ull, 0ull, 0ull};
      for (int i = tid; i < vocab; i += blockDim.x) {
        const float v = w[i];
        if (v == -INFINITY) continue;
        const unsigned long long mass = (unsigned long long)(expf(v - mx) * fixed_one);
        const unsigned int down = top_bin - (ordered_key(v) >> 24);
#pragma unroll
        for (int j = 0; j < FAST_BINS; ++j) masses[j] += down == (unsigned int)j ? mass : 0ull;
        masses[FAST_BINS] += mass;
      }
      block_sum_u64(masses, sum_scratch);
      if (tid == 0) {
        limit = (unsigned long long)((double)p_keep * (double)masses[FAST_BINS]);
        unsigned long long above = 0ull;
        for (int j = 0; j < FAST_BINS && (int)top_bin - j >= 1; ++j) {
          if (above + masses[j] > limit) {
            sel_prefix = (top_bin - j) << 24;
            sel_above = above;
            sel_found = 1;
            break;
          }
          above += masses[j];
        }
      }
      __syncthreads();
    }
    for (int shift = sel_found ? 16 : 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < HIST_COPIES * 256; b += blockDim.x) hist_copies[b] = 0ull;
      __syncthreads();
      const unsigned int prefix = sel_prefix;
      const unsigned int mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      unsigned int run_bin = 256u;  // one atomic per run of values in the same bin, as above
      unsigned long long run_mass = 0ull;
      for (int i = tid; i < vocab; i += blockDim.x) {
        const float v = w[i];
        if (v == -INFINITY) continue;
        const unsigned int key = ordered_key(v);
        if ((key & mask) != prefix) continue;
        const unsigned int bin = (key >> shift) & 255u;
        if (bin != run_bin) {
          if (run_bin < 256u) atomicAdd(&hist_copies[copy * 256 + run_bin], run_mass);
          run_bin = bin;
          run_mass = 0ull;
        }
        run_mass += (unsigned long long)(expf(v - mx) * fixed_one);
      }
      if (run_bin < 256u) atomicAdd(&hist_copies[copy * 256 + run_bin], run_mass);
      __syncthreads();
      for (int b = tid; b < 256; b += blockDim.x) {
        unsigned long long sum = 0ull;
#pragma unroll
        for (int c = 0; c < HIST_COPIES; ++c) sum += hist_copies[c * 256 + b];
        hist64[b] = sum;
      }
      __syncthreads();
      if (tid == 0) {  // `limit` lives in thread 0 alone: only it walks the histogram
        if (shift == 24) {
          unsigned long long total = 0ull;
          for (int b = 0; b < 256; ++b) total += hist64[b];
          limit = (unsigned long long)((double)p_keep * (double)total);
        }
        unsigned long long above = sel_above;
        int b = 255;
        for (; b > 0; --b) {
          if (above + hist64[b] > limit) break;
          above += hist64[b];
        }
        sel_prefix = prefix | ((unsigned int)b << shift);
        sel_above = above;
      }
      __syncthreads();
    }
    const float threshold = key_to_float(sel_prefix);
    for (int i = tid; i < vocab; i += blockDim.x)
      if (w[i] < threshold) w[i] = -INFINITY;
    __syncthreads();
  }

  // -- draw -------------------------------------------------------------------------------------
  ArgMax pick{-INFINITY, 0x7fffffff};
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = w[i];
    if (v == -INFINITY) continue;
    const float u = sample_uniform(sd, ctr, (unsigned int)i);
    pick = better(pick, ArgMax{v - logf(-logf(u)), i});
  }
  pick = block_argmax(pick, arg_scratch);
  if (tid == 0) {
    tokens[row] = pick.index;
    if (need_lse) {
      float v = penalised(x[pick.index], pick.index, pen, seen_row);
      if (pen != 1.0f && history_start) {
        const int h0 = history_start[row], h1 = history_start[row + 1];
        for (int h = h0; h < h1; ++h)
          if (history[h] == pick.index) { v = v < 0.0f ? v * pen : v / pen; break; }
      }
      logprobs[row] = v - lse;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Rows that need the filters (top-k, top-p), worked by a cluster of blocks instead of one block:
// block r of a row's cluster keeps part r of the row, divided by the temperature, in its shared
// memory; every radix pass builds a histogram per block, the blocks read one another's over
// distributed shared memory after a cluster barrier and each walks the sum (the same integers
// in every block, so they all choose the same bin).  The counts and the fixed-point masses are
// exact integers, so the ids are those of the one-block path above, which scans the row in
// global memory eleven times.  Options by state slot, as ts_sample_slots gives them; rows that
// need no filter (or are padding, or marked to be left alone) are not touched: the whole cluster
// leaves at once.
// ---------------------------------------------------------------------------------------------
#define SAMPLE_CLUSTER 8
__device__ __forceinline__ void sample_cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned int sample_remote(const void* local, int rank) {
  unsigned int remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
               : "=r"(remote) : "r"((unsigned int)__cvta_generic_to_shared(local)), "r"(rank));
  return remote;
}
__device__ __forceinline__ unsigned int sample_remote_u32(const void* local, int rank) {
  unsigned int v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(sample_remote(local, rank)));
  return v;
}
__device__ __forceinline__ unsigned long long sample_remote_u64(const void* local, int rank) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(sample_remote(local, rank)));
  return v;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, long long logits_stride, int vocab, int per,
                      const float* __restrict__ temperature, const int* __restrict__ top_k,
                      const float* __restrict__ top_p, const unsigned long long* __restrict__ seed,
                      const int* __restrict__ prompt_len, const RowLookup look,
                      int* __restrict__ tokens, const float* __restrict__ penalty,
                      const int* __restrict__ want_logprob, unsigned int* __restrict__ seen, int seen_words,
                      float* __restrict__ logprobs) {
  pdl_wait();
  extern __shared__ float w[];  // this block's part of the row: `per` values
  __shared__ ArgMax arg_scratch[33];
  __shared__ float f_scratch[33];
  __shared__ unsigned int hist32[256];        // what the others read: this block's counts per bin
  __shared__ unsigned long long hist64[256];  // and its masses per bin
  __shared__ unsigned long long total64[256];
  __shared__ unsigned int total32[256];
  __shared__ unsigned long long hist_copies[HIST_COPIES * 256];
  unsigned int* const hist_copies32 = reinterpret_cast<unsigned int*>(hist_copies);
  __shared__ float local_max, lse_max, lse_sum;
  __shared__ ArgMax local_best;
  __shared__ unsigned int sel_prefix, sel_remaining;
  __shared__ unsigned long long sel_above;

  const int row = blockIdx.y, rank = blockIdx.x, tid = threadIdx.x;  // the cluster lies along x
  const int copy = tid & (HIST_COPIES - 1);
  const int step_token = look.row_token ? look.row_token[row] : row;
  const int seq = look.seq_of_token ? look.seq_of_token[step_token] : step_token;
  if (seq < 0) return;
  const int opt = look.seq_slot[seq];
  const float temp = temperature[opt];
  const int k = top_k ? top_k[opt] : 0;
  const float p_keep = top_p ? top_p[opt] : 1.0f;
  const bool use_k = k > 0 && k < vocab, use_p = p_keep < 1.0f;
  if (!(temp > 0.0f) || (!use_k && !use_p)) return;  // not a row for this kernel (the same in every block of the cluster)
  const bool need_lse = logprobs != nullptr && want_logprob != nullptr && want_logprob[opt] != 0;
  const unsigned long long sd = seed ? seed[opt] : 0ull;
  const unsigned int ctr = (unsigned int)(look.seq_context[seq] - prompt_len[opt]);
  const float pen = penalty ? penalty[opt] : 1.0f;
  unsigned int* const seen_row = (seen && pen != 1.0f) ? seen + (size_t)opt * seen_words : nullptr;
  if (seen_row != nullptr && look.step_tokens != nullptr) {
    const int t = look.step_tokens[step_token];
    if (tid == 0 && t >= 0 && t < vocab) atomicOr(&seen_row[t >> 5], 1u << (t & 31));
    __syncthreads();
  }

  const int lo = min(vocab, rank * per), count = min(vocab, lo + per) - lo;
  const float* x = logits + (size_t)row * logits_stride + lo;
  for (int i = tid; i < count; i += blockDim.x) w[i] = penalised(x[i], lo + i, pen, seen_row) / temp;
  __syncthreads();

  // log-sum-exp of the penalised row before the temperature: every block its part, parts added in rank order
  float lse = 0.0f;
  if (need_lse) {
    float mx = -INFINITY;
    for (int i = tid; i < count; i += blockDim.x) mx = fmaxf(mx, penalised(x[i], lo + i, pen, seen_row));
    mx = block_max(mx, f_scratch);
    if (tid == 0) lse_max = mx;
    sample_cluster_barrier();
    for (int r = 0; r < SAMPLE_CLUSTER; ++r) mx = fmaxf(mx, __uint_as_float(sample_remote_u32(&lse_max, r)));
    float sum = 0.0f;
    for (int i = tid; i < count; i += blockDim.x) sum += expf(penalised(x[i], lo + i, pen, seen_row) - mx);
    sum = block_sum(sum, f_scratch);
    if (tid == 0) lse_sum = sum;
    sample_cluster_barrier();
    float total = 0.0f;
    for (int r = 0; r < SAMPLE_CLUSTER; ++r) total += __uint_as_float(sample_remote_u32(&lse_sum, r));
    lse = mx + logf(total);
  }

  if (use_k) {
    if (tid == 0) { sel_prefix = 0; sel_remaining = (unsigned int)k; }
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < HIST_COPIES * 256; b += blockDim.x) hist_copies32[b] = 0;
      __syncthreads();
      const unsigned int prefix = sel_prefix;
      const unsigned int mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < count; i += blockDim.x) {
        const unsigned int key = ordered_key(w[i]);
        if ((key & mask) != prefix) continue;
        atomicAdd(&hist_copies32[copy * 256 + ((key >> shift) & 255u)], 1u);
      }
      __syncthreads();
      for (int b = tid; b < 256; b += blockDim.x) {
        unsigned int sum = 0u;
#pragma unroll
        for (int c = 0; c < HIST_COPIES; ++c) sum += hist_copies32[c * 256 + b];
        hist32[b] = sum;
      }
      sample_cluster_barrier();  // every block's counts are in place
      for (int b = tid; b < 256; b += blockDim.x) {
        unsigned int sum = 0u;
#pragma unroll
        for (int r = 0; r < SAMPLE_CLUSTER; ++r) sum += sample_remote_u32(&hist32[b], r);
        total32[b] = sum;
      }
      __syncthreads();
      if (tid == 0) {
        unsigned int remaining = sel_remaining;
        int b = 255;
        for (; b > 0; --b) {
          if (total32[b] >= remaining) break;
          remaining -= total32[b];
        }
        sel_prefix = prefix | ((unsigned int)b << shift);
        sel_remaining = remaining;
      }
      sample_cluster_barrier();  // all have read the counts before the next pass overwrites them
    }
    const float threshold = key_to_float(sel_prefix);
    for (int i = tid; i < count; i += blockDim.x)
      if (w[i] < threshold) w[i] = -INFINITY;
    __syncthreads();
  }

  if (use_p) {
    float mx = -INFINITY;
    for (int i = tid; i < count; i += blockDim.x) mx = fmaxf(mx, w[i]);
    mx = block_max(mx, f_scratch);
    if (tid == 0) local_max = mx;
    sample_cluster_barrier();
    for (int r = 0; r < SAMPLE_CLUSTER; ++r) mx = fmaxf(mx, __uint_as_float(sample_remote_u32(&local_max, r)));
    const float fixed_one = 1099511627776.0f;  // 2^40
    if (tid == 0) { sel_prefix = 0; sel_above = 0ull; }
    unsigned long long limit = 0ull;
    __syncthreads();
    for (int shift = 24; shift >= 0; shift -= 8) {
      for (int b = tid; b < HIST_COPIES * 256; b += blockDim.x) hist_copies[b] = 0ull;
      __syncthreads();
      const unsigned int prefix = sel_prefix;
      const unsigned int mask = shift == 24 ? 0u : (0xffffffffu << (shift + 8));
      for (int i = tid; i < count; i += blockDim.x) {
        const float v = w[i];
        if (v == -INFINITY) continue;
        const unsigned int key = ordered_key(v);
        if ((key & mask) != prefix) continue;
        atomicAdd(&hist_copies[copy * 256 + ((key >> shift) & 255u)], (unsigned long long)(expf(v - mx) * fixed_one));
      }
      __syncthreads();
      for (int b = tid; b < 256; b += blockDim.x) {
        unsigned long long sum = 0ull;
#pragma unroll
        for (int c = 0; c < HIST_COPIES; ++c) sum += hist_copies[c * 256 + b];
        hist64[b] = sum;
      }
      sample_cluster_barrier();
      for (int b = tid; b < 256; b += blockDim.x) {
        unsigned long long sum = 0ull;
#pragma unroll
        for (int r = 0; r < SAMPLE_CLUSTER; ++r) sum += sample_remote_u64(&hist64[b], r);
        total64[b] = sum;
      }
      __syncthreads();
      if (tid == 0) {  // `limit` lives in thread 0 alone: only it walks the histogram
        if (shift == 24) {
          unsigned long long total = 0ull;
          for (int b = 0; b < 256; ++b) total += total64[b];
          limit = (unsigned long long)((double)p_keep * (double)total);
        }
        unsigned long long above = sel_above;
        int b = 255;
        for (; b > 0; --b) {
          if (above + total64[b] > limit) break;
          above += total64[b];
        }
        sel_prefix = prefix | ((unsigned int)b << shift);
        sel_above = above;
      }
      sample_cluster_barrier();
    }
    const float threshold = key_to_float(sel_prefix);
    for (int i = tid; i < count; i += blockDim.x)
      if (w[i] < threshold) w[i] = -INFINITY;
    __syncthreads();
  }

  ArgMax pick{-INFINITY, 0x7fffffff};
  for (int i = tid; i < count; i += blockDim.x) {
    const float v = w[i];
    if (v == -INFINITY) continue;
    const float u = sample_uniform(sd, ctr, (unsigned int)(lo + i));
    pick = better(pick, ArgMax{v - logf(-logf(u)), lo + i});
  }
  pick = block_argmax(pick, arg_scratch);
  if (tid == 0) local_best = pick;
  sample_cluster_barrier();
  if (rank == 0 && tid == 0) {
    ArgMax all{-INFINITY, 0x7fffffff};
    for (int r = 0; r < SAMPLE_CLUSTER; ++r)
      all = better(all, ArgMax{__uint_as_float(sample_remote_u32(&local_best.value, r)), (int)sample_remote_u32(&local_best.index, r)});
    tokens[row] = all.index;
    if (need_lse) logprobs[row] = penalised(logits[(size_t)row * logits_stride + all.index], all.index, pen, seen_row) - lse;
  }
  sample_cluster_barrier();  // nobody leaves while its shared memory may still be read
}

// All per-row arrays may be null, which means: greedy, no filter, no penalty, seed 0.
TS_EXPORT int ts_sample(const float* logits, long long logits_stride, float* work, int num_rows,
                        int vocab, const float* temperature, const int* top_k, const float* top_p,
                        const float* penalty, const unsigned long long* seed,
                        const unsigned int* counter, const int* history, const int* history_start,
                        int* tokens, float* logprobs, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (vocab < 1) return TS_ERR_SIZE;
  if (work == nullptr || tokens == nullptr) return TS_ERR_ARGUMENT;
  ts_launch(sample_kernel, dim3(num_rows), dim3(SAMPLE_THREADS), 0, stream, logits, logits_stride, work, vocab,
            temperature, top_k, top_p, penalty, seed, counter, history, history_start, tokens, logprobs,
            RowLookup{nullptr, nullptr, nullptr, nullptr, nullptr}, (const int*)nullptr, (int*)nullptr, 0,
            (const int*)nullptr, (unsigned int*)nullptr, 0);
  return ts_launch_status();
}

// Words of `partial` that ts_sample_slots needs for (rows, chunks).
TS_EXPORT long long ts_sample_partial_words(int num_rows, int chunks) {
  return (long long)num_rows * (4 * (long long)chunks + 1);
}

// The same with the options looked up by state slot (see the head of this file): temperature,
// top_k, top_p, seed and prompt_len are arrays over the slots, and so are penalty and
// want_logprob if given; row_token, seq_of_token, seq_slot, seq_context and step_tokens are the
// step's index arrays (RowLookup); `partial` is zeroed scratch of
// ts_sample_partial_words(num_rows, chunks) words that the kernel leaves zeroed where it
// matters, chunks >= 1.  A penalty other than 1 needs `seen` (seen_words words per slot).  A row
// whose slot wants a log-probability gets it in logprobs[row].
TS_EXPORT int ts_sample_slots(const float* logits, long long logits_stride, float* work, int num_rows,
                              int vocab, const float* temperature, const int* top_k, const float* top_p,
                              const unsigned long long* seed, const int* prompt_len, const int* row_token,
                              const int* seq_of_token, const int* seq_slot, const int* seq_context,
                              const int* step_tokens, int* tokens, int* partial, int chunks,
                              const float* penalty, const int* want_logprob, unsigned int* seen,
                              int seen_words, float* logprobs, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (vocab < 1 || chunks < 1 || chunks > 64) return TS_ERR_SIZE;
  if (work == nullptr || tokens == nullptr || seq_slot == nullptr || seq_context == nullptr || prompt_len == nullptr ||
      temperature == nullptr || partial == nullptr)
    return TS_ERR_ARGUMENT;
  if (penalty != nullptr && (seen == nullptr || seen_words < (vocab + 31) / 32)) return TS_ERR_ARGUMENT;
  if ((want_logprob != nullptr) != (logprobs != nullptr)) return TS_ERR_ARGUMENT;
  const RowLookup look{row_token, seq_of_token, seq_slot, seq_context, step_tokens};
  // rows with top-k or top-p go to a cluster of blocks that holds the row in shared memory, when it fits there
  const int per = ((vocab + SAMPLE_CLUSTER - 1) / SAMPLE_CLUSTER + 3) / 4 * 4;
  const size_t cluster_smem = (size_t)per * sizeof(float);
  const bool clustered = (top_k != nullptr || top_p != nullptr) && cluster_smem <= 180 * 1024 && num_rows <= 65535;
  ts_launch(sample_kernel, dim3(num_rows, chunks), dim3(SAMPLE_THREADS), 0, stream, logits, logits_stride, work, vocab,
            temperature, top_k, top_p, penalty, seed, (const unsigned int*)nullptr, (const int*)nullptr,
            (const int*)nullptr, tokens, logprobs, look, prompt_len, partial, clustered ? 1 : 0, want_logprob, seen,
            seen_words);
  int code = ts_launch_status();
  if (code || !clustered) return code;
  cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cluster_smem);
  ts_launch_cluster(sample_cluster_kernel, dim3(SAMPLE_CLUSTER, num_rows), dim3(SAMPLE_THREADS), cluster_smem, stream,
                    SAMPLE_CLUSTER, logits, logits_stride, vocab, per, temperature, top_k, top_p, seed, prompt_len, look,
                    tokens, penalty, want_logprob, seen, seen_words, logprobs);
  return ts_launch_status();
}

// Sets, for every token of a step whose request has a penalty other than 1, the token's bit in
// the bitmap of the request's slot: token_ids / seq_of_token per token (a negative request is
// padding), state_slots per request, penalty per slot.
__global__ void mark_seen_kernel(const int* __restrict__ token_ids, const int* __restrict__ seq_of_token,
                                 const int* __restrict__ state_slots, const float* __restrict__ penalty,
                                 unsigned int* __restrict__ seen, int seen_words, int num_tokens, int vocab) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= num_tokens) return;
  const int seq = seq_of_token[t];
  if (seq < 0) return;
  const int slot = state_slots[seq];
  const int id = token_ids[t];
  if (slot < 0 || penalty[slot] == 1.0f || id < 0 || id >= vocab) return;
  atomicOr(&seen[(size_t)slot * seen_words + (id >> 5)], 1u << (id & 31));
}

TS_EXPORT int ts_mark_seen(const int* token_ids, const int* seq_of_token, const int* state_slots,
                           const float* penalty, unsigned int* seen, int seen_words, int num_tokens,
                           int vocab, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (token_ids == nullptr || seq_of_token == nullptr || state_slots == nullptr || penalty == nullptr || seen == nullptr)
    return TS_ERR_ARGUMENT;
  if (seen_words < (vocab + 31) / 32) return TS_ERR_SIZE;
  ts_launch(mark_seen_kernel, dim3((num_tokens + 255) / 256), dim3(256), 0, stream, token_ids, seq_of_token, state_slots,
            penalty, seen, seen_words, num_tokens, vocab);
  return ts_launch_status();
}

// Plain argmax of each row (lowest id on ties); needs no scratch.
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, long long stride, int vocab,
              int* __restrict__ tokens) {
  pdl_wait();
  pdl_trigger();
  __shared__ ArgMax scratch[33];
  const float* x = logits + (size_t)blockIdx.x * stride;
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) best = better(best, ArgMax{x[i], i});
  best = block_argmax(best, scratch);
  if (threadIdx.x == 0) tokens[blockIdx.x] = best.index;
}

TS_EXPORT int ts_argmax(const float* logits, long long stride, int num_rows, int vocab,
                        int* tokens, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (vocab < 1) return TS_ERR_SIZE;
  ts_launch(argmax_kernel, dim3(num_rows), dim3(SAMPLE_THREADS), 0, stream, logits, stride, vocab, tokens);
  return ts_launch_status();
}

// The uniform that the draw uses, for a plain implementation to consume the same numbers.
TS_EXPORT float ts_sample_uniform_host(unsigned long long seed, unsigned int counter,
                                       unsigned int index) {
  return sample_uniform(seed, counter, index);
}
