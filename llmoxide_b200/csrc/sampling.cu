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
// A row of a large vocabulary is read by one SM at about 25 bytes a cycle, so what the kernel costs is how often
// it reads the row: once for the maximum, the count of finite logits and a histogram of the keys' top byte, and
// once more to collect every logit whose top byte is at least that of the k-th largest; those are usually a few
// hundred, and sorting them gives the top k with its ties in id order.  Only when they are more than 1024 (a
// row whose top logits crowd one binade) does the radix select go on byte by byte, a reading of the row each.
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

// Every element of a row to fn(value, index), four 16-byte loads in flight per thread where the row is
// 16-byte aligned.  The order in which a thread sees its elements is not the index order.
template <typename F>
__device__ __forceinline__ void scan_row(const float* __restrict__ row, int V, int tid, F&& fn) {
  if (((uintptr_t)row & 15) == 0) {
    const int n4 = V >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(row);
    int i = tid;
    for (; i + 3 * SMP_THREADS < n4; i += 4 * SMP_THREADS) {
      const float4 a = r4[i], b = r4[i + SMP_THREADS], c = r4[i + 2 * SMP_THREADS], d = r4[i + 3 * SMP_THREADS];
      const int ib = i + SMP_THREADS, ic = i + 2 * SMP_THREADS, id = i + 3 * SMP_THREADS;
      fn(a.x, 4 * i), fn(a.y, 4 * i + 1), fn(a.z, 4 * i + 2), fn(a.w, 4 * i + 3);
      fn(b.x, 4 * ib), fn(b.y, 4 * ib + 1), fn(b.z, 4 * ib + 2), fn(b.w, 4 * ib + 3);
      fn(c.x, 4 * ic), fn(c.y, 4 * ic + 1), fn(c.z, 4 * ic + 2), fn(c.w, 4 * ic + 3);
      fn(d.x, 4 * id), fn(d.y, 4 * id + 1), fn(d.z, 4 * id + 2), fn(d.w, 4 * id + 3);
    }
    for (; i < n4; i += SMP_THREADS) {
      const float4 a = r4[i];
      fn(a.x, 4 * i), fn(a.y, 4 * i + 1), fn(a.z, 4 * i + 2), fn(a.w, 4 * i + 3);
    }
    for (int j = 4 * n4 + tid; j < V; j += SMP_THREADS) fn(row[j], j);
  } else {
    for (int j = tid; j < V; j += SMP_THREADS) fn(row[j], j);
  }
}

__global__ void __launch_bounds__(SMP_THREADS, 1)
sample_kernel(float* __restrict__ logits, long long ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ repeat_penalty, const int* __restrict__ recent, int recent_width,
              const float* __restrict__ uniform, int* __restrict__ out_tokens, int* __restrict__ status) {
  __shared__ Cand cand[SMP_MAX_K];
  __shared__ unsigned hist[256];
  __shared__ unsigned hist0[256];      // the keys' top byte, over the whole row
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
  if (tid < 256) hist0[tid] = 0u;
  __syncthreads();

  const float temp = temperature[b];
  int k = top_k[b];
  const float tp = top_p[b];

  // -- argmax (also the fallback when no logit is finite), and the top byte's histogram -----
  float best = -INFINITY;
  int best_i = -1, n_finite_local = 0;
  const bool want_hist = temp > 0.f;
  scan_row(row, V, tid, [&](float v, int i) {
    if (v != v) return;
    if (finite_f32(v)) {
      ++n_finite_local;
      if (want_hist) atomicAdd(&hist0[order_key(v) >> 24], 1u);
    }
    if (best_i < 0 || v > best || (v == best && i > best_i)) { best = v; best_i = i; }
  });
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

  // ---- radix select of the k-th largest key: its top byte is in the histogram already ----------
  if (tid == 0) {
    unsigned need = (unsigned)k;
    int digit = 255;
    for (; digit > 0; --digit) {
      if (hist0[digit] >= need) break;
      need -= hist0[digit];
    }
    sh_need = need;  // how many of this digit's keys are still wanted
    sh_prefix = (unsigned)digit << 24;
    sh_count = hist0[digit];
  }
  __syncthreads();
  // every logit with at least that top byte: the ones above it (all in the top k) and the ones that share it
  const unsigned n_ge = ((unsigned)k - sh_need) + sh_count;
  const bool few = n_ge <= (unsigned)SMP_MAX_K;
  const unsigned top_byte = sh_prefix >> 24;
  unsigned mask = 0xff000000u;
  for (int shift = 16; shift >= 0 && !few; shift -= 8) {
    if (tid < 256) hist[tid] = 0u;
    __syncthreads();
    const unsigned prefix = sh_prefix;
    scan_row(row, V, tid, [&](float v, int) {
      if (!finite_f32(v)) return;
      const unsigned key = order_key(v);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    });
    __syncthreads();
    if (tid == 0) {
      unsigned need = sh_need;
      int digit = 255;
      for (; digit > 0; --digit) {
        if (hist[digit] >= need) break;
        need -= hist[digit];
      }
      sh_need = need;
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
  if (few) {
    // at most 1024 of them: all are sorted below, and the first k of the sorted order are the top k
    scan_row(row, V, tid, [&](float v, int i) {
      if (finite_f32(v) && (order_key(v) >> 24) >= top_byte) {
        const unsigned at = atomicAdd(&sh_count, 1u);
        if (at < SMP_MAX_K) { cand[at].v = v; cand[at].idx = i; }
      }
    });
  } else if (n_eq == need_eq) {
    scan_row(row, V, tid, [&](float v, int i) {
      if (finite_f32(v) && order_key(v) >= kth_key) {
        const unsigned at = atomicAdd(&sh_count, 1u);
        if (at < SMP_MAX_K) { cand[at].v = v; cand[at].idx = i; }
      }
    });
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
  const int n_gathered = min((int)sh_count, SMP_MAX_K);
  const int n_cand = min(n_gathered, k);                 // what the walk below sees: the top k
  int sort_n = 2;
  while (sort_n < n_gathered) sort_n <<= 1;
  for (int i = n_gathered + tid; i < sort_n; i += SMP_THREADS) { cand[i].v = -INFINITY; cand[i].idx = 0x7fffffff; }
  __syncthreads();

  // ---- bitonic sort: larger value first, then lower id ---------------------
  for (int size = 2; size <= sort_n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int i = tid, j = i ^ stride;
      if (j > i && j < sort_n) {
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

// Argmax alone, for greedy decoding: the last index among equal maxima.  A row is cut into slices, one CTA
// each, so that a few rows of a large vocabulary still occupy the GPU (one CTA per row reads its 600 KB one
// scalar load at a time: 30 us at eight rows).  A CTA's result is one 64-bit word, (order key of the value,
// index): the larger word is the larger value and, among equal values, the later index; 0 stands for "no
// number here".  The CTA that arrives last for a row (a counter that it sets back to 0) takes the largest of
// the slices' words.  Nothing waits for anything.
#define ARG_THREADS 256
#define ARG_MAX_ROWS 4096
#define ARG_MAX_SLICES 64
static __device__ unsigned long long g_arg_part[ARG_MAX_ROWS * ARG_MAX_SLICES];
static __device__ unsigned int g_arg_count[ARG_MAX_ROWS];

__device__ __forceinline__ unsigned long long arg_word(float v, int i) {
  return v != v ? 0ull : ((unsigned long long)order_key(v + 0.0f) << 32) | (unsigned int)i;   // (-0 counts as +0)
}

__global__ void __launch_bounds__(ARG_THREADS)
argmax_kernel(const float* __restrict__ logits, long long ld, int V, int n_slices, int slice_len,
              int* __restrict__ out_tokens) {
  __shared__ unsigned long long red[ARG_THREADS / 32];
  __shared__ bool is_last;
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y, sl = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = logits + (size_t)b * ld;
  const int lo = sl * slice_len, hi = min(V, lo + slice_len);
  unsigned long long best = 0ull;
  if ((((uintptr_t)row | (uintptr_t)(ld * 4)) & 15) == 0 && (slice_len & 3) == 0) {
    // whole groups of four, four loads in flight per thread
    const int n4 = (hi - lo) >> 2;
    const float4* r4 = reinterpret_cast<const float4*>(row + lo);
    for (int i0 = tid; i0 < n4; i0 += 4 * ARG_THREADS) {
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (i0 + u * ARG_THREADS < n4) v[u] = __ldcs(r4 + i0 + u * ARG_THREADS);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * ARG_THREADS;
        if (i < n4) {
          const int at = lo + 4 * i;
          best = max(best, arg_word(v[u].x, at));
          best = max(best, arg_word(v[u].y, at + 1));
          best = max(best, arg_word(v[u].z, at + 2));
          best = max(best, arg_word(v[u].w, at + 3));
        }
      }
    }
    for (int i = lo + 4 * n4 + tid; i < hi; i += ARG_THREADS) best = max(best, arg_word(row[i], i));
  } else {
    for (int i = lo + tid; i < hi; i += ARG_THREADS) best = max(best, arg_word(row[i], i));
  }
  for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
  if (lane == 0) red[warp] = best;
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < ARG_THREADS / 32; ++w) best = max(best, red[w]);
    if (n_slices == 1) {
      out_tokens[b] = (int)(unsigned int)best;          // (no number at all: 0)
      is_last = false;
    } else {
      g_arg_part[(size_t)b * ARG_MAX_SLICES + sl] = best;
      __threadfence();
      is_last = atomicAdd(&g_arg_count[b], 1u) == (unsigned int)(n_slices - 1);
    }
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  if (warp == 0) {
    unsigned long long all = 0ull;
    for (int i = lane; i < n_slices; i += 32) all = max(all, __ldcg(&g_arg_part[(size_t)b * ARG_MAX_SLICES + i]));
    for (int o = 16; o > 0; o >>= 1) all = max(all, __shfl_xor_sync(0xffffffffu, all, o));
    if (lane == 0) {
      out_tokens[b] = (int)(unsigned int)all;
      g_arg_count[b] = 0u;                              // for the next launch
    }
  }
}

LLMX_API int llmx_argmax(const float* logits, long long ld, int n_rows, int V, int* out_tokens,
                         cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (V <= 0 || ld < V || n_rows > 65535) return LLMX_REFUSED(1);
  // slices: about two CTAs per SM in all, each of a whole number of 4-float groups, at least 1024 floats
  int n_slices = 1;
  if (n_rows <= ARG_MAX_ROWS) {
    n_slices = (2 * 148 + n_rows - 1) / n_rows;
    if (n_slices > ARG_MAX_SLICES) n_slices = ARG_MAX_SLICES;
    if (n_slices > V / 1024) n_slices = V / 1024;
    if (n_slices < 1) n_slices = 1;
  }
  int slice_len = (V + n_slices - 1) / n_slices;
  slice_len = (slice_len + 3) & ~3;
  n_slices = (V + slice_len - 1) / slice_len;
  launch_pdl(argmax_kernel, dim3(n_slices, n_rows), dim3(ARG_THREADS), 0, stream, logits, ld, V, n_slices, slice_len,
             out_tokens);
  return LLMX_LAUNCH_STATUS();
}
