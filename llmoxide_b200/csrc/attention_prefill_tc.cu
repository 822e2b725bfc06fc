// Prompt attention on the 5th-generation tensor cores (tcgen05), head size 128,
// bfloat16, over the paged cache: variable-length batches, causal,
// grouped-query, a window or none, whole prompts or later chunks of one.
//
// Formulas as in attention.cu (crates/model/src/qwen35/cpu.rs:325-355,
// crates/model/src/cache.rs:31-37); the step's keys and values are in the cache
// before this runs (cpu.rs:314-323).
//
// A CTA owns 128 consecutive query tokens of one head (row = lane of tensor
// memory) and walks the visible keys 64 at a time (one cache page):
//   warp 0     TMA: the query tile once, then per key tile K and V, each as
//              [2 panels of 64 dims][64 keys][128 bytes], 128-byte swizzle
//   warp 1     one lane issues  S = Q K^T  (both operands K-major) into one of
//              two S buffers in tensor memory, and  O += P V  (P from tensor
//              memory, V MN-major straight from its cache layout)
//   warps 2-5  softmax, one thread per query row: tcgen05.ld the row of S,
//              mask, running maximum, exp2, row sum, P as bfloat16 back into
//              tensor memory over the scores it came from (tcgen05.st; two keys
//              to a column), where the MMA takes it as its A operand: P never
//              passes through shared memory, whose bandwidth is what a key tile
//              costs most of (Q 32 KB, K and V 16 KB each, read by the MMAs and
//              written by the copies).  O stays in tensor memory;
//              it is rescaled (load, multiply, store) only when a row's maximum
//              has grown by more than 2^8 since the maximum its exponentials
//              were taken against, which is rare after the first tiles.
// S of tile j+1 is issued before P V of tile j, so the tensor core works on the
// next scores while the softmax warps work on these.  A CTA takes half of an
// SM (96 KB of shared memory, 256 columns of tensor memory, 168 registers),
// so two CTAs share it: while one's softmax warps wait for a tensor-memory load
// or the special-function unit, the other's run.  Every mbarrier wait is
// bounded; a wait that runs out sets the status word and the CTA winds down.
#include "tc_ptx.cuh"

#define AT_ROWS 128        // query rows per CTA = MMA M
#define AT_KEYS 64         // keys per tile = MMA N of S = one cache page
#define AT_D 128
#define AT_THREADS 192        // warp 0 TMA, warp 1 MMA, warps 2..5 softmax
#define AT_PANEL (128 * 128)   // bytes of one [128 rows x 64 elements] panel of Q
#define AT_TILE (2 * AT_PANEL) // bytes of the [128 x 128] query tile
#define AT_KPANEL (AT_KEYS * 128)   // bytes of one [64 keys x 64 dims] panel of K or V
#define AT_KTILE (2 * AT_KPANEL)    // bytes of a [64 keys x 128 dims] tile of K or V
#define AT_SMEM (AT_TILE + 4 * AT_KTILE + 16 * 8 + 64)   // Q, K[2], V[2], barriers

__device__ int g_at_status = 0;    // 0, or which bounded wait ran out (1..10 below), 20: shared memory not 1024-byte aligned
__device__ __forceinline__ void at_report(int code) {
  atomicExch(&g_at_status, code);
  llmx_report(code);
}


// instruction descriptors: bf16 x bf16 -> f32, M = 128
__host__ __device__ constexpr uint32_t at_idesc(bool b_mn_major, uint32_t n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}

__global__ void __launch_bounds__(AT_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                            const int* __restrict__ block_table, int table_width, const int* __restrict__ seq_start,
                            const int* __restrict__ seq_past, int H, int G, int window, float scale_log2) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Heads run fastest in launch order and query tiles from the last one down: every head's longest tile starts
  // before any shorter one, so the work left at the end is made of short tiles.
  const int b = blockIdx.z, hq = blockIdx.x;
  const int g = hq / (H / G);
  const int tok0 = seq_start[b], n_new = seq_start[b + 1] - tok0;
  const int i0 = (gridDim.y - 1 - blockIdx.y) * AT_ROWS;
  if (i0 >= n_new) return;                                   // uniform over the CTA, before anything is set up
  const int past = seq_past[b];
  const int rows_here = min(AT_ROWS, n_new - i0);
  const int pos_lo = past + i0, pos_hi = past + i0 + rows_here - 1;
  const int first_lo = (window > 0 && pos_lo - (window - 1) > 0) ? pos_lo - (window - 1) : 0;
  const int tile_first = first_lo / AT_KEYS, tile_last = pos_hi / AT_KEYS;
  const int n_tiles = tile_last - tile_first + 1;
  const int* pages = block_table + (size_t)b * table_width;

  // shared memory: Q (32 KB), K[2], V[2] (16 KB each), then barriers
  // Half an SM leaves no room for alignment slack: the dynamic shared memory must start on a
  // 1024-byte boundary (it does when the kernel has no static shared memory); otherwise nothing runs.
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {
    if (threadIdx.x == 0) at_report(20);
    return;
  }
  uint8_t* base_ptr = smem_raw;
  const uint32_t sQ = base, sK0 = base + AT_TILE, sV0 = sK0 + 2 * AT_KTILE;
  uint8_t* pV0 = base_ptr + AT_TILE + 2 * AT_KTILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(pV0 + 2 * AT_KTILE);
  const uint32_t bar0 = smem_u32(bars);
  // s_full[st]: the scores of a tile are complete, so its K stage is free as well; pv_done[st]: P V of a tile is
  // complete, so its V stage is free, O may be rescaled and (for the last tile) read.  One commit each per tile:
  // the thread that issues the MMAs is what a CTA waits for most, and a commit costs it as much as an MMA.
  const uint32_t q_full = bar0, k_full0 = bar0 + 8, v_full0 = bar0 + 24;
  const uint32_t s_full0 = bar0 + 40, pv_done0 = bar0 + 56, p_ready = bar0 + 72;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 15);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full0 + 8u * i, 1);
      mbar_init(v_full0 + 8u * i, 1);
      mbar_init(s_full0 + 8u * i, 1);
      mbar_init(pv_done0 + 8u * i, 1);
    }
    mbar_init(p_ready, 4);                   // one arrival per softmax warp
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(256u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tS0 = tmem_base, tO = tmem_base + 2 * AT_KEYS;   // S buffers at columns 0 and 64, O at 128

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_expect_tx(q_full, AT_TILE);
      tma_load_2d(sQ, &map_q, hq * AT_D, tok0 + i0, q_full);
      tma_load_2d(sQ + AT_PANEL, &map_q, hq * AT_D + 64, tok0 + i0, q_full);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        const uint32_t parity = ((j >> 1) & 1) ^ 1;
        const int row = (pages[tile_first + j] * G + g) * LLMX_PAGE;      // the tile is one page of one kv head
        if (!mbar_wait(s_full0 + 8u * st, parity)) { at_report(1); break; }
        mbar_expect_tx(k_full0 + 8u * st, AT_KTILE);
        tma_load_2d(sK0 + (uint32_t)st * AT_KTILE, &map_k, 0, row, k_full0 + 8u * st);
        tma_load_2d(sK0 + (uint32_t)st * AT_KTILE + AT_KPANEL, &map_k, 64, row, k_full0 + 8u * st);
        if (!mbar_wait(pv_done0 + 8u * st, parity)) { at_report(2); break; }
        mbar_expect_tx(v_full0 + 8u * st, AT_KTILE);
        tma_load_2d(sV0 + (uint32_t)st * AT_KTILE, &map_v, 0, row, v_full0 + 8u * st);
        tma_load_2d(sV0 + (uint32_t)st * AT_KTILE + AT_KPANEL, &map_v, 64, row, v_full0 + 8u * st);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_s = at_idesc(false, AT_KEYS), idesc_o = at_idesc(true, AT_D);
      bool ok = mbar_wait(q_full, 0);
      if (!ok) at_report(3);
      const uint64_t q0 = umma_desc(sQ);
      auto issue_pv = [&](int j) {       // O += P_j V_j
        const int st = j & 1;
        if (!mbar_wait(p_ready, j & 1)) { at_report(5); return false; }
        if (!mbar_wait(v_full0 + 8u * st, (j >> 1) & 1)) { at_report(6); return false; }
        tc_fence_after();
        const uint64_t v0 = umma_desc_mn(sV0 + (uint32_t)st * AT_KTILE, AT_KPANEL, 1024u);
#pragma unroll
        for (int ks = 0; ks < AT_KEYS / 16; ++ks)      // 16 keys on: 2048 bytes, 128 in the descriptor's units
          umma_bf16_ts(tO, tS0 + (uint32_t)st * AT_KEYS + (uint32_t)ks * 8u, v0 + (uint64_t)(ks * 128), idesc_o,
                       (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(pv_done0 + 8u * st);
        return true;
      };
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        if (!mbar_wait(k_full0 + 8u * st, (j >> 1) & 1)) { at_report(4); ok = false; break; }
        tc_fence_after();
        const uint64_t k0 = umma_desc(sK0 + (uint32_t)st * AT_KTILE);
#pragma unroll
        for (int ks = 0; ks < AT_D / 16; ++ks) {     // (offsets in the descriptors' 16-byte units)
          const uint32_t qoff = ((uint32_t)(ks >> 2) * AT_PANEL + (uint32_t)(ks & 3) * 32u) >> 4;
          const uint32_t koff = ((uint32_t)(ks >> 2) * AT_KPANEL + (uint32_t)(ks & 3) * 32u) >> 4;
          umma_bf16(tS0 + (uint32_t)st * AT_KEYS, q0 + qoff, k0 + koff, idesc_s, ks > 0 ? 1u : 0u);
        }
        if (!(j == 0 && llmx_withhold))     // (tests: the first tile's scores are never announced)
          umma_commit(s_full0 + 8u * st);
        if (j >= 1) ok = issue_pv(j - 1);
      }
      if (ok) issue_pv(n_tiles - 1);
    }
  } else {
    // ---------------- softmax, one thread per query row ----------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int pos = past + i0 + row;                              // this row's position
    const int first = (window > 0 && pos - (window - 1) > 0) ? pos - (window - 1) : 0;
    const bool row_live = row < rows_here;
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    float m_used = -INFINITY;      // the maximum the exponentials are taken against (may lag the true one)
    float l = 0.f;                 // row sum in units of 2^-m_used
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j & 1;
      ok = mbar_wait(s_full0 + 8u * st, (j >> 1) & 1);
      if (!ok && lane == 0) at_report(7);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const uint32_t tS = tS0 + (uint32_t)st * AT_KEYS + lane_off;
      const int key0 = (tile_first + j) * AT_KEYS;
      // the row of S: four loads in flight, one wait
      uint32_t sr[AT_KEYS];
#pragma unroll
      for (int c = 0; c < AT_KEYS; c += 32) tmem_ld32_nowait(tS + (uint32_t)c, sr + c);
      tmem_ld_wait();
      // Tiles that some row of this CTA sees only in part (the diagonal, a window's edge, rows past the
      // sequence's end) are masked; the others, which is most of them, skip the compares.
      const bool edge = (key0 + AT_KEYS - 1 > pos_lo) || (window > 0 && key0 < pos_hi - (window - 1)) ||
                        (rows_here < AT_ROWS);
      if (edge) {
#pragma unroll
        for (int e = 0; e < AT_KEYS; ++e) {
          const int key = key0 + e;
          if (!(row_live && key >= first && key <= pos)) sr[e] = 0xff800000u;     // -inf
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains, so the maxima overlap
#pragma unroll
      for (int e = 0; e < AT_KEYS; e += 4) {
        mx4[0] = fmaxf(mx4[0], __uint_as_float(sr[e]));
        mx4[1] = fmaxf(mx4[1], __uint_as_float(sr[e + 1]));
        mx4[2] = fmaxf(mx4[2], __uint_as_float(sr[e + 2]));
        mx4[3] = fmaxf(mx4[3], __uint_as_float(sr[e + 3]));
      }
      const float mt = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;   // scale_log2 > 0
      // the maximum to use: keep the old one unless the true maximum outgrew it by more than 2^8
      float alpha = 1.0f;
      if (mt > m_used + 8.0f) {                                   // also the first time (m_used = -inf)
        alpha = (m_used == -INFINITY) ? 0.0f : exp2f(m_used - mt);
        m_used = mt;
      }
      l *= alpha;
      // probabilities (a masked score is -inf and gives exactly 0), their sum, and P as bfloat16 in the
      // MMA's layout: [panel = key / 64][row][128 bytes], 16-byte chunk index XOR (row % 8)
      const float neg_ref = (m_used == -INFINITY) ? 0.f : -m_used;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t packed[AT_KEYS / 2];
#pragma unroll
      for (int e = 0; e < AT_KEYS; e += 2) {
        const float p0 = ex2_approx(fmaf(__uint_as_float(sr[e]), scale_log2, neg_ref));
        const float p1 = ex2_approx(fmaf(__uint_as_float(sr[e + 1]), scale_log2, neg_ref));
        sum4[(e >> 1) & 3] += p0 + p1;
        __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
        packed[e >> 1] = *reinterpret_cast<uint32_t*>(&hh);
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // O belongs to P V of the tile before until it is done.  It is rescaled only when some row of the warp
      // needs it; otherwise P goes out first and the wait for that P V (every tile's is waited for, so that the
      // barrier's phases are followed one by one) comes after, off the path to the next P V.
      const bool rescale = j >= 1 && __any_sync(0xffffffffu, alpha != 1.0f);
      if (rescale) {
        ok = mbar_wait(pv_done0 + 8u * ((j - 1) & 1), ((j - 1) >> 1) & 1);
        if (!ok && lane == 0) at_report(8);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < AT_D; c += 32) {
          float o[32];
          tmem_ld32(tO + lane_off + (uint32_t)c, o);
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] *= alpha;
          tmem_st32(tO + lane_off + (uint32_t)c, o);
        }
      }
      // P as bfloat16 over the scores it came from: this row's lane, two keys to a column
      tmem_st32_u32(tS, packed);
      // the last tile: rows of V past the newest key were never written (or belong to another owner of the page)
      if (key0 + AT_KEYS - 1 > pos_hi) {
        ok = mbar_wait(v_full0 + 8u * st, (j >> 1) & 1);
        if (!ok && lane == 0) at_report(9);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        const int valid = pos_hi - key0 + 1;
        uint8_t* vt = pV0 + st * AT_KTILE;
        for (int idx = (warp - 2) * 32 + lane; idx < (AT_KEYS - valid) * 16; idx += 128) {
          const int r = valid + (idx >> 4), part = idx & 15;       // 16 x 16 bytes per row: 8 per panel
          *reinterpret_cast<uint4*>(vt + (part >> 3) * AT_KPANEL + r * 128 + ((part & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
      if (j >= 1 && !rescale) {
        ok = mbar_wait(pv_done0 + 8u * ((j - 1) & 1), ((j - 1) >> 1) & 1);
        if (!ok && lane == 0) at_report(8);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      }
    }
    // ---------------- normalise and store ----------------
    if (ok) {
      ok = mbar_wait(pv_done0 + 8u * ((n_tiles - 1) & 1), ((n_tiles - 1) >> 1) & 1);
      if (!ok && lane == 0) at_report(10);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    }
    if (ok) {
      tc_fence_after();
      const float inv = 1.0f / l;
      bf16* orow = out + ((size_t)(tok0 + i0 + row) * H + hq) * AT_D;
#pragma unroll 1
      for (int c = 0; c < AT_D; c += 32) {
        float o[32];
        tmem_ld32(tO + lane_off + (uint32_t)c, o);
        if (row_live) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 v;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(o[e] * inv, o[e + 1] * inv);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(o[e + 2] * inv, o[e + 3] * inv);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(o[e + 4] * inv, o[e + 5] * inv);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(o[e + 6] * inv, o[e + 7] * inv);
            v.x = *reinterpret_cast<uint32_t*>(&h0);
            v.y = *reinterpret_cast<uint32_t*>(&h1);
            v.z = *reinterpret_cast<uint32_t*>(&h2);
            v.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(orow + c + e) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
  }
}

// q, out: bf16 [T, H*128], tokens packed sequence after sequence; k_cache, v_cache: one cache entry
// [n_pages, G, 64, 128]; seq_start [B+1]; seq_past[b] = position of sequence b's first new token;
// max_new = most new tokens of a sequence.
LLMX_API int llmx_attention_prefill_tc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                       long long n_pages, const int* block_table, int table_width,
                                       const int* seq_start, const int* seq_past, int B, int T, int max_new, int H,
                                       int G, int D, int window, float scale, cudaStream_t stream) {
  if (B <= 0 || max_new <= 0 || T <= 0) return 0;
  if (D != AT_D || H <= 0 || G <= 0 || H % G || window < 0 || B > 65535 || (max_new + AT_ROWS - 1) / AT_ROWS > 65535 || n_pages <= 0)
    return LLMX_REFUSED(1);
  if (((uintptr_t)q & 15) || ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15)) return LLMX_REFUSED(1);
  CUtensorMap mq, mk, mv;
  const uint64_t cache_rows = (uint64_t)n_pages * G * LLMX_PAGE;
  if (make_map(&mq, q, (uint64_t)T, (uint64_t)H * D, (uint64_t)H * D, AT_ROWS, false)) return LLMX_REFUSED(4);
  if (make_map(&mk, k_cache, cache_rows, D, D, LLMX_PAGE, false)) return LLMX_REFUSED(4);
  if (make_map(&mv, v_cache, cache_rows, D, D, LLMX_PAGE, false)) return LLMX_REFUSED(4);
  const size_t smem = AT_SMEM;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    // all of the SM's L1 as shared memory, so that two CTAs fit
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid(H, (max_new + AT_ROWS - 1) / AT_ROWS, B);
  launch_pdl(attention_prefill_tc_kernel, grid, dim3(AT_THREADS), smem, stream, mq, mk, mv, (bf16*)out, block_table,
             table_width, seq_start, seq_past, H, G, window, scale * 1.4426950408889634f);
  return LLMX_LAUNCH_STATUS();
}

LLMX_API int llmx_attention_prefill_tc_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_at_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v) {
    int z = 0;
    cudaMemcpyToSymbol(g_at_status, &z, sizeof(int));
  }
  return v;
}
