// Next-token choice on the device, one block per sequence, over float32
// logits [B, V].  The algorithm and its order are the reference sampler's
// (crates/model/src/sample.rs:116-183): repetition penalty on the recent
// window; argmax when temperature <= 0 (the last index among equal maxima,
// sample.rs:186-192); else the k largest finite logits sorted downwards,
// p = exp((l - max) / T), the shortest prefix whose mass reaches top_p * sum,
// and a walk down that prefix with r = u * sum.  The uniform draw u comes from
// the host (one xorshift64* stream per sequence), so a sequence's tokens do not
// depend on what else is in the batch.  Equal logits are ordered by lower
// token id first.
//
// top_k in [1, 1024] runs the sorted algorithm.  top_k = 0 (no limit) with
// top_p >= 1 walks the whole vocabulary in id order instead of sorted order:
// the same distribution, another mapping from u to a token.
#include "common.cuh"

#define SMP_THREADS 1024
#define SMP_MAX_K 1024

__device__ __forceinline__ unsigned order_key(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ bool finite_f32(float v) { return fabsf(v) <= 3.402823466e38f; }

struct Cand {
  float v;
  int idx;
};
// a before b in the sorted order: larger value, then lower id
__device__ __forceinline__ bool cand_before(const Cand& a, const Cand& b) {
  return a.v > b.v || (a.v == b.v && a.idx < b.idx);
}

__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(float* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ repeat_penalty, const int* __restrict__ recent, int recent_width,
              const float* __restrict__ uniform, int* __restrict__ out_tokens, int* __restrict__ status) {
  __shared__ Cand cand[SMP_MAX_K];
  __shared__ unsigned hist[256];
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  __shared__ unsigned sh_prefix, sh_need, sh_count, sh_taken_eq;
  __shared__ int sh_result;
  __shared__ float sh_f;

  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* row = logits + (size_t)b * ld;

  // -- repetition penalty: once per occurrence, in order -------------------
  const float pen = repeat_penalty ? repeat_penalty[b] : 1.0f;
  if (pen != 1.0f && recent && tid == 0) {
    for (int i = 0; i < recent_width; ++i) {
      const int t = recent[(size_t)b * recent_width + i];
      if (t >= 0 && t < V) row[t] = row[t] > 0.f ? row[t] / pen : row[t] * pen;
    }
  }
  __syncthreads();

  const float temp = temperature[b];
  int k = top_k[b];
  const float tp = top_p[b];

  // -- argmax (also the fallback when no logit is finite) ------------------
  float best = -INFINITY;
  int best_i = -1, n_finite_local = 0;
  for (int i = tid; i < V; i += SMP_THREADS) {
    const float v = row[i];
    if (v != v) continue;
    if (finite_f32(v)) ++n_finite_local;
    if (best_i < 0 || v > best || (v == best && i > best_i)) { best = v; best_i = i; }
  }
  // reduce (value, index): larger value, then larger index
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (oi >= 0 && (best_i < 0 || ov > best || (ov == best && oi > best_i))) { best = ov; best_i = oi; }
    n_finite_local += __shfl_xor_sync(0xffffffffu, n_finite_local, o);
  }
  if (lane == 0) { red_v[warp] = best; red_i[warp] = best_i; hist[warp] = (unsigned)n_finite_local; }
  __syncthreads();
  if (warp == 0) {
    best = red_v[lane]; best_i = red_i[lane];
    int nf = (int)hist[lane];
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (oi >= 0 && (best_i < 0 || ov > best || (ov == best && oi > best_i))) { best = ov; best_i = oi; }
      nf += __shfl_xor_sync(0xffffffffu, nf, o);
    }
    if (lane == 0) { sh_result = best_i < 0 ? 0 : best_i; sh_count = (unsigned)nf; sh_f = best; }
  }
  __syncthreads();
  const int n_finite = (int)sh_count;
  const float row_max = sh_f;
  const int arg_best = sh_result;
  if (temp <= 0.f || n_finite == 0) {
    if (tid == 0) out_tokens[b] = arg_best;
    return;
  }
  const float inv_t = 1.0f / temp;
  const float u = uniform[b];

  if (k <= 0 || k >= V) {
    // ---- whole vocabulary, id order (needs top_p >= 1) -------------------
    if (tp < 1.0f && V > SMP_MAX_K) {
      if (tid == 0) { out_tokens[b] = arg_best; *(volatile int*)status = 1; }
      return;
    }
    if (V > SMP_MAX_K) {
      // Each thread owns a contiguous span of ids.  An inclusive scan of the
      // spans' masses gives every span its interval (lo, hi] of the running
      // sum; the first span with mass whose hi reaches r holds the token.
      float* pre = reinterpret_cast<float*>(cand);
      const int span = (V + SMP_THREADS - 1) / SMP_THREADS;
      const int lo_i = min(V, tid * span), hi_i = min(V, lo_i + span);
      float part = 0.f;
      for (int i = lo_i; i < hi_i; ++i) {
        const float v = row[i];
        if (finite_f32(v)) part += expf((v - row_max) * inv_t);
      }
      float incl = part;
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      if (lane == 31) red_v[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        float w = red_v[lane];
        for (int o = 1; o < 32; o <<= 1) {
          const float n = __shfl_up_sync(0xffffffffu, w, o);
          if (lane >= o) w += n;
        }
        red_v[lane] = w;
      }
      if (tid == 0) sh_result = SMP_THREADS;
      __syncthreads();
      pre[tid] = (warp ? red_v[warp - 1] : 0.f) + incl;
      __syncthreads();
      const float r = u * pre[SMP_THREADS - 1];
      if (part > 0.f && pre[tid] >= r) atomicMin(&sh_result, tid);
      __syncthreads();
      const int winner = sh_result;
      if (winner == SMP_THREADS) {  // rounding left r above every hi: the argmax stands in
        if (tid == 0) out_tokens[b] = arg_best;
        return;
      }
      if (tid == winner) {
        float acc = tid ? pre[tid - 1] : 0.f;
        int chosen = -1, last_finite = -1;
        for (int i = lo_i; i < hi_i; ++i) {
          const float v = row[i];
          if (!finite_f32(v)) continue;
          last_finite = i;
          acc += expf((v - row_max) * inv_t);
          if (acc >= r) { chosen = i; break; }
        }
        out_tokens[b] = chosen >= 0 ? chosen : last_finite;
      }
      return;
    }
    k = V;  // small vocabulary: the sorted algorithm covers it
  }
  if (k > SMP_MAX_K) {
    if (tid == 0) { out_tokens[b] = arg_best; *(volatile int*)status = 2; }
    return;
  }
  if (k > n_finite) k = n_finite;

  // ---- radix select of the k-th largest key ------------------------------
  if (tid == 0) { sh_prefix = 0u; sh_need = (unsigned)k; }
  __syncthreads();
  unsigned mask = 0u;
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) hist[tid] = 0u;
    __syncthreads();
    const unsigned prefix = sh_prefix;
    for (int i = tid; i < V; i += SMP_THREADS) {
      const float v = row[i];
      if (!finite_f32(v)) continue;
      const unsigned key = order_key(v);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      unsigned need = sh_need;
      int digit = 255;
      for (; digit > 0; --digit) {
        if (hist[digit] >= need) break;
        need -= hist[digit];
      }
      sh_need = need;  // how many of this digit's keys are still wanted
      sh_prefix = prefix | ((unsigned)digit << shift);
      sh_count = hist[digit];
    }
    __syncthreads();
    mask |= 255u << shift;
  }
  const unsigned kth_key = sh_prefix;
  const unsigned need_eq = sh_need;      // keys equal to the k-th that belong to the top k
  const unsigned n_eq = sh_count;        // keys equal to the k-th in the row

  // ---- gather the candidates ---------------------------------------------
  __syncthreads();  // every thread has read the select's results before they are reset
  if (tid == 0) { sh_count = 0u; sh_taken_eq = 0u; }
  __syncthreads();
  if (n_eq == need_eq) {
    for (int i = tid; i < V; i += SMP_THREADS) {
      const float v = row[i];
      if (finite_f32(v) && order_key(v) >= kth_key) {
        const unsigned at = atomicAdd(&sh_count, 1u);
        if (at < SMP_MAX_K) { cand[at].v = v; cand[at].idx = i; }
      }
    }
  } else {
    // ties at the threshold: those with the lowest ids are kept, so the equal
    // keys are taken in id order, one chunk of the row at a time
    for (int base = 0; base < V; base += SMP_THREADS) {
      const int i = base + tid;
      const float v = i < V ? row[i] : 0.f;
      const bool fin = i < V && finite_f32(v);
      const unsigned key = fin ? order_key(v) : 0u;
      if (fin && key > kth_key) {
        const unsigned at = atomicAdd(&sh_count, 1u);
        if (at < SMP_MAX_K) { cand[at].v = v; cand[at].idx = i; }
      }
      const bool eq = fin && key == kth_key;
      const unsigned ball = __ballot_sync(0xffffffffu, eq);
      __syncthreads();
      if (lane == 0) hist[warp] = __popc(ball);
      __syncthreads();
      unsigned before = sh_taken_eq;
      for (int w = 0; w < warp; ++w) before += hist[w];
      const unsigned rank = before + __popc(ball & ((1u << lane) - 1u));
      if (eq && rank < need_eq) {
        const unsigned at = atomicAdd(&sh_count, 1u);
        if (at < SMP_MAX_K) { cand[at].v = v; cand[at].idx = i; }
      }
      __syncthreads();
      if (tid == 0) {
        unsigned total = 0;
        for (int w = 0; w < SMP_THREADS / 32; ++w) total += hist[w];
        sh_taken_eq += total;
      }
      __syncthreads();
    }
  }
  __syncthreads();
  const int n_cand = min((int)sh_count, SMP_MAX_K);
  for (int i = n_cand + tid; i < SMP_MAX_K; i += SMP_THREADS) { cand[i].v = -INFINITY; cand[i].idx = 0x7fffffff; }
  __syncthreads();

  // ---- bitonic sort: larger value first, then lower id ---------------------
  for (int size = 2; size <= SMP_MAX_K; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int i = tid, j = i ^ stride;
      if (j > i) {
        const bool up = (i & size) == 0;
        const Cand a = cand[i], c = cand[j];
        const bool swap = up ? cand_before(c, a) : cand_before(a, c);
        if (swap) { cand[i] = c; cand[j] = a; }
      }
      __syncthreads();
    }
  }

  // ---- probabilities, nucleus, walk: sequential, as the reference sums ----
  if (tid == 0) {
    const float mx = cand[0].v;
    float sum = 0.f;
    for (int i = 0; i < n_cand; ++i) {
      const float p = expf((cand[i].v - mx) * inv_t);
      cand[i].v = p;
      sum += p;
    }
    int cutoff = n_cand;
    if (tp < 1.0f) {
      const float target = tp * sum;
      float acc = 0.f;
      for (int i = 0; i < n_cand; ++i) {
        acc += cand[i].v;
        if (acc >= target) { cutoff = i + 1; break; }
      }
      sum = 0.f;
      for (int i = 0; i < cutoff; ++i) sum += cand[i].v;
    }
    float r = u * sum;
    int chosen = cand[cutoff - 1].idx;
    for (int i = 0; i < cutoff; ++i) {
      r -= cand[i].v;
      if (r <= 0.f) { chosen = cand[i].idx; break; }
    }
    out_tokens[b] = chosen;
  }
}

LLMX_API int llmx_sample(float* logits, long long ld, int n_rows, int V, const float* temperature,
                         const int* top_k, const float* top_p, const float* repeat_penalty, const int* recent,
                         int recent_width, const float* uniform, int* out_tokens, int* status,
                         cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0 || ld < V || !temperature || !top_k || !top_p || !uniform || !out_tokens || !status)
    return LLMX_REFUSED(1);
  launch_pdl(sample_kernel, dim3(n_rows), dim3(SMP_THREADS), 0, stream, logits, ld, V, temperature, top_k, top_p, repeat_penalty,
                                                     recent, recent_width, uniform, out_tokens, status);
  return LLMX_LAUNCH_STATUS();
}

// Argmax alone, for greedy decoding: the last index among equal maxima.
__global__ void __launch_bounds__(SMP_THREADS)
argmax_kernel(const float* __restrict__ logits, long long ld, int V, int* __restrict__ out_tokens) {
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)b * ld;
  float best = -INFINITY;
  int best_i = -1;
  for (int i = tid; i < V; i += SMP_THREADS) {
    const float v = row[i];
    if (v != v) continue;
    if (best_i < 0 || v > best || (v == best && i > best_i)) { best = v; best_i = i; }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (oi >= 0 && (best_i < 0 || ov > best || (ov == best && oi > best_i))) { best = ov; best_i = oi; }
  }
  if (lane == 0) { red_v[warp] = best; red_i[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = red_v[lane]; best_i = red_i[lane];
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (oi >= 0 && (best_i < 0 || ov > best || (ov == best && oi > best_i))) { best = ov; best_i = oi; }
    }
    if (lane == 0) out_tokens[b] = best_i < 0 ? 0 : best_i;
  }
}

LLMX_API int llmx_argmax(const float* logits, long long ld, int n_rows, int V, int* out_tokens,
                         cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0 || ld < V) return LLMX_REFUSED(1);
  launch_pdl(argmax_kernel, dim3(n_rows), dim3(SMP_THREADS), 0, stream, logits, ld, V, out_tokens);
  return LLMX_LAUNCH_STATUS();
}
