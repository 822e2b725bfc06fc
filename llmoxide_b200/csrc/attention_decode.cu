// Decode attention over the paged bfloat16 cache: one new token per sequence,
// the key range split across CTAs ("splitting the key range across workgroups
// and reducing the partials afterwards" is the fix the reference's authors
// name for their own decode attention, crates/gpu/src/shaders/attn.wgsl:13-17).
//
// Formulas as in attention.cu (crates/model/src/qwen35/cpu.rs:325-355): kv
// head g = hq / (H/G); keys first..p visible, first = 0 or p-(w-1); scores
// scaled; softmax with the maximum subtracted; all in float32.
//
// Work split.  grid = (chunks, G * head_groups, B).  A CTA has 4 warps and
// owns one sequence, one kv head, up to 4 of the query heads that share it,
// and a chunk of 4 * pages_per_warp cache pages; a warp walks its pages one
// at a time.  Within a page of 64 keys a warp takes 4 keys per iteration: 8
// lanes per key, each lane D/8 contiguous dims, so a key row is read once,
// 16 bytes per lane, and feeds every query head of the group.  Scores of a
// page go to shared memory; the page's maximum updates the running maximum
// once, so the accumulators are rescaled per page and not per key.  The four
// lane groups and then the four warps are merged at the end, and the CTA
// writes an unnormalised partial (max, sum, acc) to the workspace; a second
// kernel merges the chunks of each (sequence, head).
#include "common.cuh"

#define DEC_WARPS 4
#define DEC_MAX_HEADS 4                      // query heads per CTA
#define DEC_KEYS_PER_ITER 4
#define DEC_LANES_PER_KEY 8

template <int D>
struct DecTraits {
  static constexpr int DIMS = D / DEC_LANES_PER_KEY;   // contiguous dims per lane
};

// loads DIMS consecutive bf16 starting at p (aligned to DIMS * 2 bytes) into float
template <int DIMS>
__device__ __forceinline__ void load_dims(const bf16* __restrict__ p, float* out) {
  if constexpr (DIMS % 8 == 0) {
#pragma unroll
    for (int i = 0; i < DIMS / 8; ++i) {
      const uint4 raw = *reinterpret_cast<const uint4*>(p + 8 * i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        out[8 * i + 2 * j] = f.x;
        out[8 * i + 2 * j + 1] = f.y;
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < DIMS / 2; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + 2 * i));
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  }
}

template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                        const int* __restrict__ block_table, int table_width, const int* __restrict__ seq_past,
                        float* __restrict__ ws, int H, int G, int window, float scale, int pages_per_warp,
                        int n_chunks) {
  constexpr int DIMS = DecTraits<D>::DIMS;
  __shared__ float sc[DEC_WARPS][DEC_MAX_HEADS][LLMX_PAGE];      // scores, then probabilities, of a warp's page
  __shared__ float merge_acc[DEC_WARPS][DEC_MAX_HEADS][D];
  __shared__ float merge_ml[DEC_WARPS][DEC_MAX_HEADS][2];

  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane >> 3;            // which of the 4 keys of an iteration
  const int part = lane & 7;            // which slice of the head's dims
  const int chunk = blockIdx.x, b = blockIdx.z;
  const int R = H / G;
  const int head_groups = (R + DEC_MAX_HEADS - 1) / DEC_MAX_HEADS;
  const int g = blockIdx.y / head_groups, hg = blockIdx.y % head_groups;
  const int h0 = g * R + hg * DEC_MAX_HEADS;                      // first query head of this CTA
  const int n_heads = min(DEC_MAX_HEADS, R - hg * DEC_MAX_HEADS);

  const int p = seq_past[b];                                      // position of the new token
  const int first = (window > 0 && p - (window - 1) > 0) ? p - (window - 1) : 0;
  const int first_page = first / LLMX_PAGE, last_page = p / LLMX_PAGE;
  const int* pages = block_table + (size_t)b * table_width;

  // queries of this CTA's heads, this lane's dims, pre-scaled
  float qr[DEC_MAX_HEADS][DIMS];
#pragma unroll
  for (int h = 0; h < DEC_MAX_HEADS; ++h) {
    if (h < n_heads) {
      load_dims<DIMS>(q + ((size_t)b * H + h0 + h) * D + part * DIMS, qr[h]);
#pragma unroll
      for (int i = 0; i < DIMS; ++i) qr[h][i] *= scale;
    } else {
#pragma unroll
      for (int i = 0; i < DIMS; ++i) qr[h][i] = 0.f;
    }
  }
  float acc[DEC_MAX_HEADS][DIMS];
  float m[DEC_MAX_HEADS], l[DEC_MAX_HEADS];
#pragma unroll
  for (int h = 0; h < DEC_MAX_HEADS; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < DIMS; ++i) acc[h][i] = 0.f;
  }

  const int page_lo = first_page + (chunk * DEC_WARPS + warp) * pages_per_warp;
  for (int pi = 0; pi < pages_per_warp; ++pi) {
    const int lp = page_lo + pi;                                  // logical page (warp-uniform)
    if (lp > last_page) break;
    const int phys = pages[lp];
    const bf16* kpage = k_cache + cache_row_offset(phys, g, 0, G, D);
    const bf16* vpage = v_cache + cache_row_offset(phys, g, 0, G, D);
    const int key0 = lp * LLMX_PAGE;

    // ---- scores of the page ------------------------------------------------
#pragma unroll 4
    for (int it = 0; it < LLMX_PAGE / DEC_KEYS_PER_ITER; ++it) {
      const int r = it * DEC_KEYS_PER_ITER + sub;
      const int key = key0 + r;
      float kv[DIMS];
      load_dims<DIMS>(kpage + (size_t)r * D + part * DIMS, kv);
      float s[DEC_MAX_HEADS];
#pragma unroll
      for (int h = 0; h < DEC_MAX_HEADS; ++h) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < DIMS; ++i) d = fmaf(qr[h][i], kv[i], d);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        s[h] = d;
      }
      const bool visible = key >= first && key <= p;
      if (part < DEC_MAX_HEADS) {
        // lane `part` of the key's group stores head `part` (no divergent register index)
        float mine = s[0];
#pragma unroll
        for (int h = 1; h < DEC_MAX_HEADS; ++h) mine = (part == h) ? s[h] : mine;
        sc[warp][part][r] = visible ? mine : -INFINITY;
      }
    }
    __syncwarp();

    // ---- page maximum, probabilities, sums ------------------------------------
#pragma unroll
    for (int h = 0; h < DEC_MAX_HEADS; ++h) {
      const float s0 = sc[warp][h][lane], s1 = sc[warp][h][lane + 32];
      const float pm = warp_max(fmaxf(s0, s1));
      const float m_new = fmaxf(m[h], pm);                        // finite: every page walked has a visible key
      const float corr = __expf(m[h] - m_new);
      const float p0 = __expf(s0 - m_new), p1 = __expf(s1 - m_new);
      sc[warp][h][lane] = p0;
      sc[warp][h][lane + 32] = p1;
      l[h] = l[h] * corr + warp_sum(p0 + p1);
      m[h] = m_new;
#pragma unroll
      for (int i = 0; i < DIMS; ++i) acc[h][i] *= corr;
    }
    __syncwarp();

    // ---- values --------------------------------------------------------------------
#pragma unroll 4
    for (int it = 0; it < LLMX_PAGE / DEC_KEYS_PER_ITER; ++it) {
      const int r = it * DEC_KEYS_PER_ITER + sub;
      float vv[DIMS];
      load_dims<DIMS>(vpage + (size_t)r * D + part * DIMS, vv);
#pragma unroll
      for (int h = 0; h < DEC_MAX_HEADS; ++h) {
        const float w = sc[warp][h][r];
        if (w != 0.f) {      // a masked row may hold anything, even NaN; its weight is exactly 0
#pragma unroll
          for (int i = 0; i < DIMS; ++i) acc[h][i] = fmaf(w, vv[i], acc[h][i]);
        }
      }
    }
    __syncwarp();
  }

  // ---- merge the 4 key groups of the warp (they share m and l) -----------------
#pragma unroll
  for (int h = 0; h < DEC_MAX_HEADS; ++h)
#pragma unroll
    for (int i = 0; i < DIMS; ++i) {
      float a = acc[h][i];
      a += __shfl_xor_sync(0xffffffffu, a, 8);
      a += __shfl_xor_sync(0xffffffffu, a, 16);
      acc[h][i] = a;
    }
  if (sub == 0) {
#pragma unroll
    for (int h = 0; h < DEC_MAX_HEADS; ++h)
#pragma unroll
      for (int i = 0; i < DIMS; ++i) merge_acc[warp][h][part * DIMS + i] = acc[h][i];
  }
  if (lane == 0) {
#pragma unroll
    for (int h = 0; h < DEC_MAX_HEADS; ++h) {
      merge_ml[warp][h][0] = m[h];
      merge_ml[warp][h][1] = l[h];
    }
  }
  __syncthreads();

  // ---- merge the warps and write the chunk's partial ------------------------------
  // workspace layout: [B][H][n_chunks][D + 2] = (acc[D], max, sum)
  for (int idx = threadIdx.x; idx < n_heads * D; idx += DEC_WARPS * 32) {
    const int h = idx / D, d = idx % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mx = fmaxf(mx, merge_ml[w][h][0]);
    float a = 0.f, ls = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float mw = merge_ml[w][h][0];
      const float f = (mw == -INFINITY) ? 0.f : __expf(mw - mx);
      a += f * merge_acc[w][h][d];
      ls += f * merge_ml[w][h][1];
    }
    float* dst = ws + (((size_t)b * H + h0 + h) * n_chunks + chunk) * (D + 2);
    dst[d] = a;
    if (d == 0) {
      dst[D] = mx;
      dst[D + 1] = ls;
    }
  }
}

// Merges the chunk partials of each (sequence, head): out = sum_c e^(m_c - m) acc_c / sum_c e^(m_c - m) l_c.
__global__ void attention_decode_merge_kernel(const float* __restrict__ ws, bf16* __restrict__ out, int H, int D,
                                              int n_chunks) {
  pdl_launch_dependents();
  pdl_wait();
  const int bh = blockIdx.x;
  const float* base = ws + (size_t)bh * n_chunks * (D + 2);
  float mx = -INFINITY;
  for (int c = 0; c < n_chunks; ++c) mx = fmaxf(mx, base[(size_t)c * (D + 2) + D]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f, l = 0.f;
    for (int c = 0; c < n_chunks; ++c) {
      const float* pc = base + (size_t)c * (D + 2);
      const float mc = pc[D];
      if (mc == -INFINITY) continue;       // a chunk beyond this sequence's keys
      const float f = __expf(mc - mx);
      a += f * pc[d];
      l += f * pc[D + 1];
    }
    out[(size_t)bh * D + d] = __float2bfloat16_rn(a / l);
  }
}

template <int D>
static int launch_decode(const void* q, void* out, const void* k_cache, const void* v_cache, const int* block_table,
                         int table_width, const int* seq_past, float* ws, int B, int H, int G, int window,
                         float scale, int pages_per_warp, int n_chunks, cudaStream_t stream) {
  const int R = H / G;
  const int head_groups = (R + DEC_MAX_HEADS - 1) / DEC_MAX_HEADS;
  dim3 grid(n_chunks, G * head_groups, B);
  launch_pdl(attention_decode_kernel<D>, grid, dim3(DEC_WARPS * 32), 0, stream,
      (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, block_table, table_width, seq_past, ws, H, G,
      window, scale, pages_per_warp, n_chunks);
  int rc = LLMX_LAUNCH_STATUS();
  if (rc) return rc;
  launch_pdl(attention_decode_merge_kernel, dim3(B * H), dim3(D <= 64 ? 64 : 128), 0, stream, (const float*)ws,
             (bf16*)out, H, D, n_chunks);
  return LLMX_LAUNCH_STATUS();
}

// q, out: bf16 [B, H*D] (one token per sequence, in batch order); seq_past[b] = the token's position.
// ws: float32 workspace of B*H*n_chunks*(D+2) elements.  A chunk is 4 * pages_per_warp pages of 64 keys;
// n_chunks chunks must cover the longest visible key range of the batch.
LLMX_API int llmx_attention_decode(const void* q, void* out, const void* k_cache, const void* v_cache,
                                   const int* block_table, int table_width, const int* seq_past, float* ws, int B,
                                   int H, int G, int D, int window, float scale, int pages_per_warp, int n_chunks,
                                   cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || window < 0 || pages_per_warp < 1 || n_chunks < 1 || !ws) return LLMX_REFUSED(1);
  if (B > 65535 || (long long)G * ((H / G + DEC_MAX_HEADS - 1) / DEC_MAX_HEADS) > 65535) return LLMX_REFUSED(3);
#define CASE(DD)                                                                                               \
  case DD:                                                                                                     \
    return launch_decode<DD>(q, out, k_cache, v_cache, block_table, table_width, seq_past, ws, B, H, G, window, \
                             scale, pages_per_warp, n_chunks, stream)
  switch (D) {
    CASE(16); CASE(32); CASE(48); CASE(64); CASE(80); CASE(96); CASE(112); CASE(128);
    CASE(144); CASE(160); CASE(176); CASE(192); CASE(208); CASE(224); CASE(240); CASE(256);
    default: return LLMX_REFUSED(1);
  }
#undef CASE
}
