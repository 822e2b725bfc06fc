// Decode attention over the paged bfloat16 cache: one new token per sequence,
// the key range split across CTAs ("splitting the key range across workgroups
// and reducing the partials afterwards" is the fix the reference's authors
// name for their own decode attention, crates/gpu/src/shaders/attn.wgsl:13-17).
//
// Formulas as in attention.cu (crates/model/src/qwen35/cpu.rs:325-355): kv
// head g = hq / (H/G); keys first..p visible, first = 0 or p-(w-1); scores
// scaled; softmax with the maximum subtracted; statistics in float32.
//
// Work split.  grid = (chunks, G * head_groups, B).  A CTA has 2 warps and
// owns one sequence, one kv head, up to 16 of the query heads that share it
// (the rows of one m16n8k16 tile; unused rows are zero), and a chunk of
// 2 * pages_per_warp cache pages.  Each warp walks its pages in tiles of 32
// keys: cp.async brings the tile's keys and values (contiguous in a page) to
// the warp's own three-stage shared-memory ring, so the next two tiles are in
// flight while this one is multiplied; scores and the weighted sum run on the tensor
// cores.  Rows are padded by 16 bytes so that ldmatrix is free of bank
// conflicts at every head size.  The two warps are merged through shared
// memory and the CTA writes one unnormalised partial (acc, max, sum) per head
// to the workspace; a second kernel merges the chunks of each (sequence, head).
#include "common.cuh"

#define DEC_WARPS 2
#define DEC_ROWS 16                          // query heads per CTA = rows of the MMA tile
#define DEC_TILE 32                          // keys per pipeline stage
#define DEC_STAGES 3

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D>
struct DecSmem {
  static constexpr int ROW = D * 2 + 16;                         // padded row, bytes
  static constexpr int TILE = DEC_TILE * ROW;                    // one K or V tile
  static constexpr int Q = DEC_ROWS * ROW;
  static constexpr int WARP = Q + DEC_STAGES * 2 * TILE;         // per warp: Q, then (K, V) per stage
  static constexpr int TOTAL = DEC_WARPS * WARP;
};

template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                        const int* __restrict__ block_table, int table_width, const int* __restrict__ seq_past,
                        float* __restrict__ ws, bf16* __restrict__ out, int H, int G, int window, float scale_log2,
                        int pages_per_warp, int n_chunks) {
  using S = DecSmem<D>;
  constexpr int CHUNKS = D / 8;            // 16-byte chunks per row
  constexpr int KSTEPS = D / 16;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_launch_dependents();
  pdl_wait();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int chunk = blockIdx.x, b = blockIdx.z;
  const int R = H / G;
  const int head_groups = (R + DEC_ROWS - 1) / DEC_ROWS;
  const int g = blockIdx.y / head_groups, hg = blockIdx.y % head_groups;
  const int h0 = g * R + hg * DEC_ROWS;                          // first query head of this CTA
  const int n_heads = min(DEC_ROWS, R - hg * DEC_ROWS);

  const int p = seq_past[b];                                      // position of the new token
  const int first = (window > 0 && p - (window - 1) > 0) ? p - (window - 1) : 0;
  const int* pages = block_table + (size_t)b * table_width;

  uint8_t* wsm = smem + warp * S::WARP;
  const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(wsm);
  const uint32_t sKV = sQ + S::Q;

  // this warp's tiles of 32 keys: from its first page to its last, clipped to the visible keys
  const int page_lo = first / LLMX_PAGE + (chunk * DEC_WARPS + warp) * pages_per_warp;
  const int tile_lo = max(page_lo * (LLMX_PAGE / DEC_TILE), first / DEC_TILE);
  const int tile_hi = min((page_lo + pages_per_warp) * (LLMX_PAGE / DEC_TILE) - 1, p / DEC_TILE);
  const int n_tiles = tile_hi - tile_lo + 1;                      // <= 0: nothing to do

  auto load_tile = [&](int tile, int stage) {
    const int key0 = tile * DEC_TILE;
    const int phys = pages[key0 / LLMX_PAGE];
    const size_t off = cache_row_offset(phys, g, key0 % LLMX_PAGE, G, D);
    const uint32_t sK = sKV + stage * 2 * S::TILE, sV = sK + S::TILE;
    for (int idx = lane; idx < DEC_TILE * CHUNKS; idx += 32) {
      const int r = idx / CHUNKS, c = idx % CHUNKS;
      cp_async16(sK + r * S::ROW + c * 16, k_cache + off + (size_t)r * D + c * 8);
      cp_async16(sV + r * S::ROW + c * 16, v_cache + off + (size_t)r * D + c * 8);
    }
  };

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;     // rows lane/4 and lane/4 + 8

  if (n_tiles > 0) {
    // queries: rows = heads of the group, zero beyond n_heads
    for (int idx = lane; idx < DEC_ROWS * CHUNKS; idx += 32) {
      const int r = idx / CHUNKS, c = idx % CHUNKS;
      if (r < n_heads) cp_async16(sQ + r * S::ROW + c * 16, q + ((size_t)b * H + h0 + r) * D + c * 8);
      else *reinterpret_cast<uint4*>(wsm + r * S::ROW + c * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
    // ring of DEC_STAGES tiles: one commit group per tile slot (empty past the end), so that
    // "all but the newest DEC_STAGES - 1 groups are done" always means "tile t has landed"
    for (int i = 0; i < DEC_STAGES - 1; ++i) {
      if (i < n_tiles) load_tile(tile_lo + i, i);
      cp_async_commit();
    }

    for (int t = 0; t < n_tiles; ++t) {
      const int stage = t % DEC_STAGES;
      if (t + DEC_STAGES - 1 < n_tiles) load_tile(tile_lo + t + DEC_STAGES - 1, (t + DEC_STAGES - 1) % DEC_STAGES);
      cp_async_commit();
      cp_async_wait<DEC_STAGES - 1>();
      __syncwarp();
      const uint32_t sK = sKV + stage * 2 * S::TILE, sV = sK + S::TILE;
      const int key0 = (tile_lo + t) * DEC_TILE;
      if (key0 + DEC_TILE - 1 > p) {
        // rows past the newest key were never written by this sequence: weight 0, but 0 * NaN is NaN
        uint8_t* vt = wsm + S::Q + stage * 2 * S::TILE + S::TILE;
        const int valid = p - key0 + 1;
        for (int idx = lane; idx < (DEC_TILE - valid) * CHUNKS; idx += 32) {
          const int r = valid + idx / CHUNKS, c = idx % CHUNKS;
          *reinterpret_cast<uint4*>(vt + r * S::ROW + c * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
      }

      // ---- S = Q K^T : 16 x 32 ------------------------------------------------------
      float s[DEC_TILE / 8][4];
#pragma unroll
      for (int j = 0; j < DEC_TILE / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(sQ + (lane & 15) * S::ROW + (2 * ks + (lane >> 4)) * 16, a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int jp = 0; jp < DEC_TILE / 16; ++jp) {
          uint32_t b0, b1, b2, b3;
          const int kr = jp * 16 + (lane & 7) + ((lane >> 4) << 3);
          const int kc = 2 * ks + ((lane >> 3) & 1);
          ldmatrix_x4(sK + kr * S::ROW + kc * 16, b0, b1, b2, b3);
          mma_bf16(s[2 * jp], a, b0, b1);
          mma_bf16(s[2 * jp + 1], a, b2, b3);
        }
      }

      // ---- mask, running maximum, probabilities -------------------------------------------
      float mx0 = m0, mx1 = m1;
#pragma unroll
      for (int j = 0; j < DEC_TILE / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + 8 * j + 2 * (lane & 3) + e;
          const bool vis = key >= first && key <= p;
          s[j][e] = vis ? s[j][e] * scale_log2 : -INFINITY;
          s[j][2 + e] = vis ? s[j][2 + e] * scale_log2 : -INFINITY;
          mx0 = fmaxf(mx0, s[j][e]);
          mx1 = fmaxf(mx1, s[j][2 + e]);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float c0 = exp2f(m0 - mx0), c1 = exp2f(m1 - mx1);     // every tile walked has a visible key
      m0 = mx0;
      m1 = mx1;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pf[DEC_TILE / 16][4];
#pragma unroll
      for (int j = 0; j < DEC_TILE / 8; ++j) {
        const float e0 = exp2f(s[j][0] - mx0), e1 = exp2f(s[j][1] - mx0);
        const float e2 = exp2f(s[j][2] - mx1), e3 = exp2f(s[j][3] - mx1);
        sum0 += e0 + e1;
        sum1 += e2 + e3;
        pf[j >> 1][(j & 1) * 2] = pack_bf16(e0, e1);
        pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(e2, e3);
      }
      l0 = l0 * c0 + sum0;
      l1 = l1 * c1 + sum1;
#pragma unroll
      for (int j = 0; j < D / 8; ++j) {
        o[j][0] *= c0;
        o[j][1] *= c0;
        o[j][2] *= c1;
        o[j][3] *= c1;
      }

      // ---- O += P V ------------------------------------------------------------------------------
#pragma unroll
      for (int kk = 0; kk < DEC_TILE / 16; ++kk) {
#pragma unroll
        for (int jp = 0; jp < D / 16; ++jp) {
          uint32_t b0, b1, b2, b3;
          const int vr = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int vc = 2 * jp + (lane >> 4);
          ldmatrix_x4_trans(sV + vr * S::ROW + vc * 16, b0, b1, b2, b3);
          mma_bf16(o[2 * jp], pf[kk], b0, b1);
          mma_bf16(o[2 * jp + 1], pf[kk], b2, b3);
        }
      }
      __syncwarp();   // the stage is refilled by the next iteration's loads
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  }

  // ---- merge the warps and write the chunk's partial ------------------------------------------
  // The pipeline buffers are done with; they are reused as [warp][row][D] accumulators and
  // [warp][row][2] statistics.  workspace layout: [B][H][n_chunks][D + 2] = (acc[D], max, sum)
  __syncthreads();
  float* macc = reinterpret_cast<float*>(smem);                                  // [DEC_WARPS][DEC_ROWS][D]
  float* mml = macc + DEC_WARPS * DEC_ROWS * D;                                  // [DEC_WARPS][DEC_ROWS][2]
  {
    const int r0 = lane >> 2, r1 = r0 + 8;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      const int col = 8 * j + 2 * (lane & 3);
      float* a0 = macc + ((size_t)warp * DEC_ROWS + r0) * D + col;
      float* a1 = macc + ((size_t)warp * DEC_ROWS + r1) * D + col;
      a0[0] = o[j][0];
      a0[1] = o[j][1];
      a1[0] = o[j][2];
      a1[1] = o[j][3];
    }
    if ((lane & 3) == 0) {
      mml[(warp * DEC_ROWS + r0) * 2] = m0;
      mml[(warp * DEC_ROWS + r0) * 2 + 1] = l0;
      mml[(warp * DEC_ROWS + r1) * 2] = m1;
      mml[(warp * DEC_ROWS + r1) * 2 + 1] = l1;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_heads * D; idx += DEC_WARPS * 32) {
    const int h = idx / D, d = idx % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mx = fmaxf(mx, mml[(w * DEC_ROWS + h) * 2]);
    float a = 0.f, ls = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float mw = mml[(w * DEC_ROWS + h) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mx);
      a += f * macc[((size_t)w * DEC_ROWS + h) * D + d];
      ls += f * mml[(w * DEC_ROWS + h) * 2 + 1];
    }
    if (n_chunks == 1) {
      out[((size_t)b * H + h0 + h) * D + d] = __float2bfloat16_rn(a / ls);   // nothing to merge with
    } else {
      float* dst = ws + (((size_t)b * H + h0 + h) * n_chunks + chunk) * (D + 2);
      dst[d] = a;
      if (d == 0) {
        dst[D] = mx;
        dst[D + 1] = ls;
      }
    }
  }
}

// Merges the chunk partials of each (sequence, head): out = sum_c 2^(m_c - m) acc_c / sum_c 2^(m_c - m) l_c
// (the maxima are in the base-2 domain of the scores).
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
      const float f = exp2f(mc - mx);
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
  const int head_groups = (R + DEC_ROWS - 1) / DEC_ROWS;
  dim3 grid(n_chunks, G * head_groups, B);
  size_t smem = DecSmem<D>::TOTAL;
  const size_t merge = (size_t)DEC_WARPS * DEC_ROWS * (D + 2) * sizeof(float);
  if (merge > smem) smem = merge;
  auto kernel = attention_decode_kernel<D>;
  static bool attr_set = false;
  if (!attr_set && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  launch_pdl(kernel, grid, dim3(DEC_WARPS * 32), smem, stream, (const bf16*)q, (const bf16*)k_cache,
             (const bf16*)v_cache, block_table, table_width, seq_past, ws, (bf16*)out, H, G, window,
             scale * 1.4426950408889634f, pages_per_warp, n_chunks);
  int rc = LLMX_LAUNCH_STATUS();
  if (rc || n_chunks == 1) return rc;
  launch_pdl(attention_decode_merge_kernel, dim3(B * H), dim3(D <= 64 ? 64 : 128), 0, stream, (const float*)ws,
             (bf16*)out, H, D, n_chunks);
  return LLMX_LAUNCH_STATUS();
}

// q, out: bf16 [B, H*D] (one token per sequence, in batch order); seq_past[b] = the token's position.
// ws: float32 workspace of B*H*n_chunks*(D+2) elements.  A chunk is 2 * pages_per_warp pages of 64 keys;
// n_chunks chunks must cover the longest visible key range of the batch.
LLMX_API int llmx_attention_decode(const void* q, void* out, const void* k_cache, const void* v_cache,
                                   const int* block_table, int table_width, const int* seq_past, float* ws, int B,
                                   int H, int G, int D, int window, float scale, int pages_per_warp, int n_chunks,
                                   cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || window < 0 || pages_per_warp < 1 || n_chunks < 1 || (n_chunks > 1 && !ws))
    return LLMX_REFUSED(1);
  if (B > 65535 || (long long)G * ((H / G + DEC_ROWS - 1) / DEC_ROWS) > 65535) return LLMX_REFUSED(3);
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

// ---------------------------------------------------------------------------
// The same kernels for callers that must not allocate: the workspace is a
// file-scope device array.  See attention_decode_noalloc.h for who needs this
// and for the rules (size limit, first call outside capture, shared array).
// ---------------------------------------------------------------------------
#include "attention_decode_noalloc.h"

static __device__ __align__(256) float g_noalloc_workspace[LLMX_NOALLOC_WS_FLOATS];

// In host code the array's name is only a handle for the runtime, not an address a kernel can use:
// the device address is asked for once per device, with that device current, and kept.
#define LLMX_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[LLMX_NOALLOC_MAX_DEVICES];

LLMX_API int llmx_attention_decode_noalloc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                           const int* block_table, int table_width, const int* seq_past, int B,
                                           int H, int G, int D, int window, float scale, int pages_per_warp,
                                           int n_chunks, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || D <= 0 || n_chunks < 1) return LLMX_REFUSED(1);
  const unsigned long long need = (unsigned long long)B * H * n_chunks * (unsigned long long)(D + 2);
  if (need > LLMX_NOALLOC_WS_FLOATS) return LLMX_NOALLOC_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= LLMX_NOALLOC_MAX_DEVICES) return LLMX_REFUSED(3);
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_workspace);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  return llmx_attention_decode(q, out, k_cache, v_cache, block_table, table_width, seq_past, g_noalloc_ptr[dev], B,
                               H, G, D, window, scale, pages_per_warp, n_chunks, stream);
}
