// Attention over the paged cache, general form: any number of heads and
// groups, any head size that is a multiple of 16 up to 256, a window or none,
// whole prompts and single tokens alike.  It is the float32 path's kernel and
// the bfloat16 path's fallback for the sizes the tiled kernels refuse.
//
// For the query at position p of head hq (crates/model/src/qwen35/cpu.rs:325-355):
// kv head g = hq / (H/G); keys first..p are visible, first = 0 or p-(w-1) under
// a window (crates/model/src/cache.rs:31-37); s_j = (q . k_j) * scale; softmax
// with the maximum subtracted; out = sum_j w_j v_j.  All of it in float32.
//
// One warp per (token, head).  Keys are taken 32 at a time starting at
// `first`: lane j scores key first + c*32 + j with a sequential dot over D,
// the chunk's maximum and sum update a running softmax, and the lanes then
// own dims (lane, lane+32, ...) of the output and add the chunk's values key
// by key.  Chunk boundaries depend on (first, p) only, so a position's result
// does not depend on how tokens were cut into steps or batched.
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_MAX_D 256

template <typename TA, typename TC>
__global__ void attention_paged_kernel(const TA* __restrict__ q, TA* __restrict__ out,
                                       const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                                       const int* __restrict__ block_table, int table_width,
                                       const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                       int H, int G, int D, int window, float scale) {
  extern __shared__ float q_buf[];  // [ATT_WARPS][D]
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;                        // tokens on x: a step may bring more than 65535
  const int hq = blockIdx.y * ATT_WARPS + warp;
  if (hq >= H) return;
  const int g = hq / (H / G);
  const int p = token_pos[t];
  const int first = (window > 0 && p - (window - 1) > 0) ? p - (window - 1) : 0;
  const int* pages = block_table + (size_t)token_seq[t] * table_width;

  float* qs = q_buf + warp * D;
  const TA* qrow = q + ((size_t)t * H + hq) * D;
  for (int i = lane; i < D; i += 32) qs[i] = to_f32(qrow[i]);
  __syncwarp();

  constexpr int MAX_OWN = ATT_MAX_D / 32;
  float acc[MAX_OWN];
#pragma unroll
  for (int i = 0; i < MAX_OWN; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int base = first; base <= p; base += 32) {
    const int j = base + lane;
    const bool live = j <= p;
    float s = -INFINITY;
    if (live) {
      const TC* krow = k_cache + cache_row_offset(pages[j / LLMX_PAGE], g, j % LLMX_PAGE, G, D);
      float dot = 0.f;
      for (int i = 0; i < D; ++i) dot += qs[i] * to_f32(krow[i]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first chunk; lane 0 is always live
    const float e = live ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(e);
#pragma unroll
    for (int i = 0; i < MAX_OWN; ++i) acc[i] *= corr;
    const int n_live = (p - base + 1) < 32 ? (p - base + 1) : 32;
    for (int jj = 0; jj < n_live; ++jj) {
      const float w = __shfl_sync(0xffffffffu, e, jj);
      const int key = base + jj;
      const TC* vrow = v_cache + cache_row_offset(pages[key / LLMX_PAGE], g, key % LLMX_PAGE, G, D);
#pragma unroll
      for (int i = 0; i < MAX_OWN; ++i) {
        const int dim = lane + 32 * i;
        if (dim < D) acc[i] += w * to_f32(vrow[dim]);
      }
    }
    m = m_new;
  }
  const float inv = 1.0f / l;
  TA* orow = out + ((size_t)t * H + hq) * D;
#pragma unroll
  for (int i = 0; i < MAX_OWN; ++i) {
    const int dim = lane + 32 * i;
    if (dim < D) orow[dim] = from_f32<TA>(acc[i] * inv);
  }
}

LLMX_API int llmx_attention_paged(const void* q, void* out, int act_dtype, const void* k_cache,
                                  const void* v_cache, int cache_dtype, const int* block_table, int table_width,
                                  const int* token_seq, const int* token_pos, int n_tokens, int H, int G, int D,
                                  int window, float scale, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || D > ATT_MAX_D || window < 0) return LLMX_REFUSED(1);
  dim3 grid(n_tokens, (H + ATT_WARPS - 1) / ATT_WARPS);
  const size_t smem = (size_t)ATT_WARPS * D * sizeof(float);
#define CASE(TA, TC)                                                                                      \
  launch_pdl(attention_paged_kernel<TA, TC>, grid, dim3(ATT_WARPS * 32), smem, stream,                    \
      (const TA*)q, (TA*)out, (const TC*)k_cache, (const TC*)v_cache, block_table, table_width, token_seq, \
      token_pos, H, G, D, window, scale)
  if (act_dtype == LLMX_F32 && cache_dtype == LLMX_F32) CASE(float, float);
  else if (act_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) CASE(bf16, bf16);
  else if (act_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) CASE(float, bf16);
  else if (act_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) CASE(bf16, float);
  else return LLMX_REFUSED(2);
#undef CASE
  return LLMX_LAUNCH_STATUS();
}
