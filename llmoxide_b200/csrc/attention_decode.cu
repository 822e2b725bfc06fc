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
// owns one sequence, one kv head, up to 8 of the query heads that share it,
// and one of n_chunks equal shares of THAT sequence's visible keys: the number
// of chunks comes from the batch's shape, the share from the sequence's own
// length on the device, so every warp of a sequence walks the same number of
// tiles however long the block table is.
//
// A warp walks its tiles of 32 keys through its own three-stage shared-memory
// ring, each stage with an mbarrier, so the next two tiles are in flight while
// this one is multiplied.  At head sizes that are multiples of 64 one lane
// asks the copy engine for the whole tile (tensor copies of 32 rows x 64 head
// dims, laid down with the 128-byte swizzle); at the others every lane copies
// 16-byte pieces with cp.async into padded rows.  Either layout keeps ldmatrix
// free of bank conflicts.
//
// The products are taken transposed, keys and head dims on the 16-wide M axis
// of mma.sync m16n8k16 and the (few) query heads on the 8-wide N axis:
// S^T = K Q^T and O^T = V^T P^T.  With 4 heads per kv head half of N is
// padding, where heads on M would leave three quarters of it idle, and the
// softmax touches 8 numbers per lane and tile.  P^T reaches the second
// product's operand layout through movmatrix.
//
// What does not depend on the kernel before (lengths, block table, keys and
// values of earlier steps) is read ahead of the programmatic-launch wait, so
// the first tiles stream while the kernel that wrote q and the new key still
// runs; only the tile that holds the new token's row waits.
//
// The two warps are merged through shared memory into one unnormalised
// partial (acc, max, sum) per head.  With up to 8 chunks the CTAs of one
// (sequence, kv head, head group) form a thread-block cluster and merge their
// partials out of each other's shared memory, each CTA a slice of the output:
// no workspace, no trip through global memory.  With more chunks the partials
// go to a workspace, and the CTA that arrives last at the group's counter
// merges them and leaves the counter at zero for the next launch.  Either way
// the chunks are summed in chunk order, so the result does not depend on
// timing.
#include "tc_ptx.cuh"

#define DEC_WARPS 2
#define DEC_ROWS 8                           // query heads per CTA = the N of one MMA tile
#define DEC_TILE 32                          // keys per pipeline stage
#define DEC_STAGES 3
#define DEC_MAX_CHUNKS 32                    // shares of one sequence's keys
#define DEC_WS_ROW(D) ((D) + 4)              // a partial in the workspace: acc[D], max, sum, 2 unused (rows stay 16-byte aligned)
#define DEC_PANEL (DEC_TILE * 128)           // a tile's 64 head dims as the tensor copy lays them down: 128-byte rows

static __device__ int g_dec_status;          // 0; 1 after a copy that never completed; 2: shared memory not 1024-byte aligned
__device__ __forceinline__ void dec_report(int code) {
  atomicExch(&g_dec_status, code);
  llmx_report(code);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// This thread's copies so far count as one arrival at the barrier once they have landed.
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
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
// The transpose of an 8x8 matrix of 16-bit elements held one 32-bit word per lane (row lane/4, columns 2(lane%4)+{0,1}).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Two layouts of a tile in shared memory, both free of ldmatrix bank conflicts.  Head sizes that are multiples
// of 64 come by tensor copies (one request per 64 head dims of a tile, issued by one lane) in panels of
// 128-byte rows with the hardware's 128-byte swizzle.  The other head sizes come by 16-byte cp.async of every
// lane into rows padded by 16 bytes.
template <int D>
struct DecSmem {
  static constexpr bool TMA = D % 64 == 0;
  static constexpr int ROW = D * 2 + 16;                                     // padded row, bytes (cp.async layout)
  static constexpr int TILE = TMA ? (D / 64) * DEC_PANEL : DEC_TILE * ROW;   // one K or V tile
  static constexpr int WARP = DEC_STAGES * 2 * TILE;                         // per warp: (K, V) per stage
  static constexpr int BARS = DEC_WARPS * WARP;                              // then one mbarrier per warp and stage
  static constexpr int TOTAL = BARS + DEC_WARPS * DEC_STAGES * 8 + 16;
  // byte offset of 16-byte chunk c of row r within a tile
  __device__ static __forceinline__ uint32_t at(int r, int c) {
    if (TMA) return (uint32_t)((c >> 3) * DEC_PANEL + r * 128 + (((c & 7) ^ (r & 7)) << 4));
    return (uint32_t)(r * ROW + c * 16);
  }
};

template <int D>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                        const int* __restrict__ block_table, int table_width, const int* __restrict__ seq_past,
                        float* __restrict__ ws, unsigned int* __restrict__ counters, bf16* __restrict__ out, int H,
                        int G, int window, float scale_log2, int n_chunks, int cluster_merge) {
  using S = DecSmem<D>;
  constexpr int KSTEPS = D / 16;
  constexpr uint32_t TILE_BYTES = 2u * DEC_TILE * D * 2u;        // what one stage's copies bring
  extern __shared__ __align__(1024) uint8_t smem[];
  int& s_last = *reinterpret_cast<int*>(smem + S::BARS + DEC_WARPS * DEC_STAGES * 8);
  pdl_launch_dependents();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gq = lane >> 2, tq = lane & 3;                        // the MMA fragments' row group and column pair
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
  const uint32_t sKV = (uint32_t)__cvta_generic_to_shared(wsm);
  const bool misaligned = S::TMA && (sKV & 1023u);   // the swizzled layout is a function of the address: refuse, never guess
  if (misaligned && threadIdx.x == 0) dec_report(2);
  const uint32_t bars = (uint32_t)__cvta_generic_to_shared(smem + S::BARS) + warp * DEC_STAGES * 8;
  if (lane == 0) {
    // a tensor copy's bytes are counted against one announcement; cp.async counts one arrival per lane
    for (int i = 0; i < DEC_STAGES; ++i) mbar_init(bars + 8 * i, S::TMA ? 1 : 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (S::TMA) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
  }
  __syncwarp();

  // this warp's tiles of 32 keys: an equal share of the sequence's visible tiles
  const int t_first = first / DEC_TILE, t_last = p / DEC_TILE;
  const int per_warp = (t_last - t_first + n_chunks * DEC_WARPS) / (n_chunks * DEC_WARPS);   // ceil(tiles / warps)
  const int tile_lo = t_first + (chunk * DEC_WARPS + warp) * per_warp;
  const int tile_hi = min(tile_lo + per_warp - 1, t_last);
  const int n_tiles = misaligned ? 0 : tile_hi - tile_lo + 1;     // <= 0: nothing to do

  const bool withhold = llmx_withhold != 0;       // tests: the first CTA's first warp never asks for its first tile
  auto load_tile = [&](int tile, int stage) {
    if (withhold && tile == tile_lo && warp == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) return;
    const int key0 = tile * DEC_TILE;
    const int phys = pages[key0 / LLMX_PAGE];
    const uint32_t sK = sKV + stage * 2 * S::TILE, sV = sK + S::TILE, bar = bars + 8 * stage;
    if (S::TMA) {
      if (lane == 0) {
        const int row = (phys * G + g) * LLMX_PAGE + key0 % LLMX_PAGE;      // the tile's first row of [rows, D]
        mbar_expect_tx(bar, TILE_BYTES);
#pragma unroll
        for (int pn = 0; pn < D / 64; ++pn) {
          tma_load_2d(sK + pn * DEC_PANEL, &map_k, 64 * pn, row, bar);
          tma_load_2d(sV + pn * DEC_PANEL, &map_v, 64 * pn, row, bar);
        }
      }
    } else {
      constexpr int CHUNKS = D / 8;
      const size_t off = cache_row_offset(phys, g, key0 % LLMX_PAGE, G, D);
      for (int idx = lane; idx < DEC_TILE * CHUNKS; idx += 32) {
        const int r = idx / CHUNKS, c = idx % CHUNKS;
        cp_async16(sK + S::at(r, c), k_cache + off + (size_t)r * D + c * 8);
        cp_async16(sV + S::at(r, c), v_cache + off + (size_t)r * D + c * 8);
      }
      cp_async_arrive(bar);
    }
  };

  float o[D / 16][4];                                             // O^T: head dims 16j + gq (+8), heads 2tq, 2tq+1
#pragma unroll
  for (int j = 0; j < D / 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;     // heads 2tq and 2tq + 1

  // Tiles before the new token's own are complete since earlier steps: they start now.
  int issued = 0;
  for (; issued < DEC_STAGES - 1 && issued < n_tiles && tile_lo + issued < t_last; ++issued)
    load_tile(tile_lo + issued, issued);
  pdl_wait();

  if (n_tiles > 0) {
    for (; issued < DEC_STAGES - 1 && issued < n_tiles; ++issued) load_tile(tile_lo + issued, issued);
    // Q^T as the B operand of every k-step: head gq, head dims 16ks + 2tq (+1) and + 8
    uint32_t qb[KSTEPS][2];
    {
      const uint32_t* qrow = reinterpret_cast<const uint32_t*>(q + ((size_t)b * H + h0 + min(gq, n_heads - 1)) * D);
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const uint32_t lo = __ldcg(qrow + 8 * ks + tq), hi = __ldcg(qrow + 8 * ks + 4 + tq);
        qb[ks][0] = gq < n_heads ? lo : 0u;
        qb[ks][1] = gq < n_heads ? hi : 0u;
      }
    }

    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int stage = t % DEC_STAGES;
      if (issued < n_tiles) {                                     // the stage read in the iteration before is free again
        load_tile(tile_lo + issued, issued % DEC_STAGES);
        ++issued;
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bars + 8 * stage, (t / DEC_STAGES) & 1));   // the warp leaves together
      if (!ok) break;
      const uint32_t sK = sKV + stage * 2 * S::TILE, sV = sK + S::TILE;
      const int key0 = (tile_lo + t) * DEC_TILE;
      if (key0 + DEC_TILE - 1 > p) {
        // rows past the newest key were never written by this sequence: weight 0, but 0 * NaN is NaN
        uint8_t* vt = wsm + stage * 2 * S::TILE + S::TILE;
        const int valid = p - key0 + 1;
        for (int idx = lane; idx < (DEC_TILE - valid) * (D / 8); idx += 32) {
          const int r = valid + idx / (D / 8), c = idx % (D / 8);
          *reinterpret_cast<uint4*>(vt + S::at(r, c)) = make_uint4(0u, 0u, 0u, 0u);
        }
        __syncwarp();
      }

      // ---- S^T = K Q^T : 32 keys x 8 heads ----------------------------------------------------------
      float s[DEC_TILE / 16][4];                                 // keys 16i + gq (+8), heads 2tq, 2tq+1
#pragma unroll
      for (int i = 0; i < DEC_TILE / 16; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int i = 0; i < DEC_TILE / 16; ++i) {
          uint32_t a0, a1, a2, a3;
          ldmatrix_x4(sK + S::at(16 * i + (lane & 15), 2 * ks + (lane >> 4)), a0, a1, a2, a3);
          mma_bf16(s[i], a0, a1, a2, a3, qb[ks][0], qb[ks][1]);
        }
      }

      // ---- mask, running maximum, probabilities -------------------------------------------------------
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < DEC_TILE / 16; ++i) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {                              // rows gq and gq + 8
          const int key = key0 + 16 * i + gq + 8 * e;
          const bool vis = key >= first && key <= p;
          s[i][2 * e] = vis ? s[i][2 * e] * scale_log2 : -INFINITY;
          s[i][2 * e + 1] = vis ? s[i][2 * e + 1] * scale_log2 : -INFINITY;
          mx0 = fmaxf(mx0, s[i][2 * e]);
          mx1 = fmaxf(mx1, s[i][2 * e + 1]);
        }
      }
#pragma unroll
      for (int sh = 4; sh < 32; sh <<= 1) {                        // over the lanes that hold the same heads
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, sh));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, sh));
      }
      mx0 = fmaxf(mx0, m0);                                        // every tile walked has a visible key
      mx1 = fmaxf(mx1, m1);
      const float c0 = exp2f(m0 - mx0), c1 = exp2f(m1 - mx1);
      m0 = mx0;
      m1 = mx1;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pb[DEC_TILE / 16][2];                              // P^T as the B operand: keys 2tq (+1) and + 8, head gq
#pragma unroll
      for (int i = 0; i < DEC_TILE / 16; ++i) {
        const float e0 = exp2f(s[i][0] - mx0), e1 = exp2f(s[i][1] - mx1);
        const float e2 = exp2f(s[i][2] - mx0), e3 = exp2f(s[i][3] - mx1);
        sum0 += e0 + e2;
        sum1 += e1 + e3;
        pb[i][0] = movmatrix_trans(pack_bf16(e0, e1));
        pb[i][1] = movmatrix_trans(pack_bf16(e2, e3));
      }
      l0 = l0 * c0 + sum0;
      l1 = l1 * c1 + sum1;
#pragma unroll
      for (int j = 0; j < D / 16; ++j) {
        o[j][0] *= c0;
        o[j][1] *= c1;
        o[j][2] *= c0;
        o[j][3] *= c1;
      }

      // ---- O^T += V^T P^T ------------------------------------------------------------------------------
#pragma unroll
      for (int i = 0; i < DEC_TILE / 16; ++i) {
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
          uint32_t a0, a1, a2, a3;
          const int vr = 16 * i + (lane & 7) + ((lane >> 4) << 3);
          const int vc = 2 * j + ((lane >> 3) & 1);
          ldmatrix_x4_trans(sV + S::at(vr, vc), a0, a1, a2, a3);
          mma_bf16(o[j], a0, a1, a2, a3, pb[i][0], pb[i][1]);
        }
      }
      __syncwarp();   // the stage is refilled by the next iteration's copies
    }
    if (!ok && lane == 0) dec_report(1);
    if (!S::TMA) asm volatile("cp.async.wait_all;" ::: "memory");
#pragma unroll
    for (int sh = 4; sh < 32; sh <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, sh);
      l1 += __shfl_xor_sync(0xffffffffu, l1, sh);
    }
  }

  // ---- merge the warps and write the chunk's partial ------------------------------------------
  // The pipeline buffers are done with; they are reused as [warp][row][D] accumulators and
  // [warp][row][2] statistics.  workspace layout: [B][H][n_chunks][D + 4] = (acc[D], max, sum, -, -)
  __syncthreads();
  float* macc = reinterpret_cast<float*>(smem);                                  // [DEC_WARPS][DEC_ROWS][D]
  float* mml = macc + DEC_WARPS * DEC_ROWS * D;                                  // [DEC_WARPS][DEC_ROWS][2]
  float* cacc = mml + DEC_WARPS * DEC_ROWS * 2;                                  // [DEC_ROWS][D]  the CTA's partial,
  float* cml = cacc + DEC_ROWS * D;                                              // [DEC_ROWS][2]  for its cluster
  {
    const int hA = 2 * tq, hB = hA + 1;
#pragma unroll
    for (int j = 0; j < D / 16; ++j) {
      const int d0 = 16 * j + gq;
      macc[((size_t)warp * DEC_ROWS + hA) * D + d0] = o[j][0];
      macc[((size_t)warp * DEC_ROWS + hB) * D + d0] = o[j][1];
      macc[((size_t)warp * DEC_ROWS + hA) * D + d0 + 8] = o[j][2];
      macc[((size_t)warp * DEC_ROWS + hB) * D + d0 + 8] = o[j][3];
    }
    if (gq == 0) {
      mml[(warp * DEC_ROWS + hA) * 2] = m0;
      mml[(warp * DEC_ROWS + hA) * 2 + 1] = l0;
      mml[(warp * DEC_ROWS + hB) * 2] = m1;
      mml[(warp * DEC_ROWS + hB) * 2 + 1] = l1;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_heads * (D / 4); idx += DEC_WARPS * 32) {     // four dims at a time
    const int h = idx / (D / 4), d = (idx % (D / 4)) * 4;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) mx = fmaxf(mx, mml[(w * DEC_ROWS + h) * 2]);
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    float ls = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float mw = mml[(w * DEC_ROWS + h) * 2];
      const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mx);
      const float4 v = *reinterpret_cast<const float4*>(macc + ((size_t)w * DEC_ROWS + h) * D + d);
      a.x += f * v.x;
      a.y += f * v.y;
      a.z += f * v.z;
      a.w += f * v.w;
      ls += f * mml[(w * DEC_ROWS + h) * 2 + 1];
    }
    if (n_chunks == 1) {                                                              // nothing to merge with
      __nv_bfloat162 lo = __floats2bfloat162_rn(a.x / ls, a.y / ls), hi = __floats2bfloat162_rn(a.z / ls, a.w / ls);
      *reinterpret_cast<uint2*>(out + ((size_t)b * H + h0 + h) * D + d) =
          make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    } else if (cluster_merge) {
      *reinterpret_cast<float4*>(cacc + (size_t)h * D + d) = a;
      if (d == 0) {
        cml[2 * h] = mx;
        cml[2 * h + 1] = ls;
      }
    } else {
      float* dst = ws + (((size_t)b * H + h0 + h) * n_chunks + chunk) * DEC_WS_ROW(D);
      __stcg(reinterpret_cast<float4*>(dst + d), a);
      if (d == 0) {
        __stcg(dst + D, mx);
        __stcg(dst + D + 1, ls);
      }
    }
  }
  if (n_chunks == 1) return;

  if (cluster_merge) {
    // ---- the cluster's CTAs (rank = chunk) each merge a slice of the outputs out of all ranks' shared memory ----
    // out = sum_c 2^(m_c - m) acc_c / sum_c 2^(m_c - m) l_c   (the maxima are in the base-2 domain)
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    const uint32_t my_acc = (uint32_t)__cvta_generic_to_shared(cacc), my_ml = (uint32_t)__cvta_generic_to_shared(cml);
    const int groups = n_heads * (D / 4), per = (groups + n_chunks - 1) / n_chunks;
    const int hi = min(groups, (chunk + 1) * per);
    for (int idx = chunk * per + threadIdx.x; idx < hi; idx += DEC_WARPS * 32) {
      const int h = idx / (D / 4), d = (idx % (D / 4)) * 4;
      // every rank's statistics and its four accumulators of this slice are asked for together: one trip
      // through the cluster's shared memory, not two
      float mc[8], lc[8], mx = -INFINITY;
      float4 vc[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        mc[c] = -INFINITY;
        lc[c] = 0.f;
        vc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < n_chunks) {
          uint32_t ra, rb;
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(my_ml + 8u * h), "r"(c));
          asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(rb) : "r"(my_acc + 4u * (h * D + d)), "r"(c));
          asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(mc[c]), "=f"(lc[c]) : "r"(ra));
          asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                       : "=f"(vc[c].x), "=f"(vc[c].y), "=f"(vc[c].z), "=f"(vc[c].w)
                       : "r"(rb));
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) mx = fmaxf(mx, mc[c]);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      float l = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < n_chunks && mc[c] != -INFINITY) {            // -inf: a chunk that got none of the keys
          const float w = exp2f(mc[c] - mx);
          a.x += w * vc[c].x;
          a.y += w * vc[c].y;
          a.z += w * vc[c].z;
          a.w += w * vc[c].w;
          l += w * lc[c];
        }
      }
      const float r = 1.f / l;
      __nv_bfloat162 lo = __floats2bfloat162_rn(a.x * r, a.y * r), hi2 = __floats2bfloat162_rn(a.z * r, a.w * r);
      uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi2));
      *reinterpret_cast<uint2*>(out + ((size_t)b * H + h0 + h) * D + d) = packed;
    }
    // nobody leaves while another CTA may still read its shared memory
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    return;
  }

  // ---- the last CTA of this (sequence, kv head, head group) merges the chunks ------------------
  // out = sum_c 2^(m_c - m) acc_c / sum_c 2^(m_c - m) l_c   (the maxima are in the base-2 domain)
  __syncthreads();                          // every thread's partials are written ...
  if (threadIdx.x == 0) {
    // ... and this release (cumulative over what the barrier ordered before it) publishes them with the arrival
    unsigned int* ctr = counters + (size_t)b * gridDim.y + blockIdx.y;
    unsigned int arrived;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(arrived) : "l"(ctr) : "memory");
    s_last = (arrived == (unsigned int)n_chunks - 1u);
    if (s_last) *ctr = 0u;                 // every CTA of the group has arrived: ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  // per (head, chunk): the factor 2^(m_c - m), and per head 1 / sum_c factor * l_c  (in the pipeline buffers, free now)
  float* fac = reinterpret_cast<float*>(smem);                   // [DEC_ROWS][DEC_MAX_CHUNKS]
  float* lsum = fac + DEC_ROWS * DEC_MAX_CHUNKS;                 // [DEC_ROWS][DEC_MAX_CHUNKS]
  float* inv = lsum + DEC_ROWS * DEC_MAX_CHUNKS;                 // [DEC_ROWS]
  const float* base = ws + ((size_t)b * H + h0) * n_chunks * DEC_WS_ROW(D);
  for (int idx = threadIdx.x; idx < n_heads * n_chunks; idx += DEC_WARPS * 32) {
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(base + (size_t)idx * DEC_WS_ROW(D) + D));
    fac[(idx / n_chunks) * DEC_MAX_CHUNKS + idx % n_chunks] = ml.x;
    lsum[(idx / n_chunks) * DEC_MAX_CHUNKS + idx % n_chunks] = ml.y;
  }
  __syncthreads();
  if (threadIdx.x < n_heads) {
    float* f = fac + threadIdx.x * DEC_MAX_CHUNKS;
    const float* ls = lsum + threadIdx.x * DEC_MAX_CHUNKS;
    float mx = -INFINITY;
    for (int c = 0; c < n_chunks; ++c) mx = fmaxf(mx, f[c]);
    float l = 0.f;
    for (int c = 0; c < n_chunks; ++c) {
      const float w = (f[c] == -INFINITY) ? 0.f : exp2f(f[c] - mx);   // -inf: a chunk that got none of the keys
      f[c] = w;
      if (w != 0.f) l += w * ls[c];
    }
    inv[threadIdx.x] = 1.f / l;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_heads * (D / 4); idx += DEC_WARPS * 32) {
    const int h = idx / (D / 4), d = (idx % (D / 4)) * 4;
    const float* row = base + (size_t)h * n_chunks * DEC_WS_ROW(D) + d;
    const float* f = fac + h * DEC_MAX_CHUNKS;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int c = 0; c < n_chunks; ++c) {
      const float w = f[c];
      float4 v = __ldcg(reinterpret_cast<const float4*>(row + (size_t)c * DEC_WS_ROW(D)));
      if (w != 0.f) {                      // an unused chunk's row may hold anything
        a.x += w * v.x;
        a.y += w * v.y;
        a.z += w * v.z;
        a.w += w * v.w;
      }
    }
    const float r = inv[h];
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x * r, a.y * r), hi = __floats2bfloat162_rn(a.z * r, a.w * r);
    uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    *reinterpret_cast<uint2*>(out + ((size_t)b * H + h0 + h) * D + d) = packed;
  }
}

template <int D>
static int launch_decode(const void* q, void* out, const void* k_cache, const void* v_cache, long long n_pages,
                         const int* block_table, int table_width, const int* seq_past, float* ws, unsigned int* counters, int B, int H, int G,
                         int window, float scale, int n_chunks, cudaStream_t stream) {
  const int R = H / G;
  const int head_groups = (R + DEC_ROWS - 1) / DEC_ROWS;
  dim3 grid(n_chunks, G * head_groups, B);
  size_t smem = DecSmem<D>::TOTAL;
  size_t merge = (size_t)(DEC_WARPS + 1) * DEC_ROWS * (D + 2) * sizeof(float);
  if (merge < (size_t)DEC_ROWS * (2 * DEC_MAX_CHUNKS + 1) * sizeof(float)) merge = (size_t)DEC_ROWS * (2 * DEC_MAX_CHUNKS + 1) * sizeof(float);
  if (merge > smem) smem = merge;
  auto kernel = attention_decode_kernel<D>;
  static bool attr_set = false;
  if (!attr_set && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  CUtensorMap mk, mv;
  memset(&mk, 0, sizeof(mk));
  memset(&mv, 0, sizeof(mv));
  if (DecSmem<D>::TMA) {
    const uint64_t cache_rows = (uint64_t)n_pages * G * LLMX_PAGE;
    if (make_map(&mk, k_cache, cache_rows, D, D, DEC_TILE, false)) return LLMX_REFUSED(4);
    if (make_map(&mv, v_cache, cache_rows, D, D, DEC_TILE, false)) return LLMX_REFUSED(4);
  }
  // up to 8 chunks (the portable cluster size): merged inside a cluster, nothing goes through the workspace
  const int cluster_merge = (n_chunks > 1 && n_chunks <= 8) ? 1 : 0;
  if (cluster_merge)
    launch_pdl_cluster(kernel, grid, dim3(DEC_WARPS * 32), smem, stream, (unsigned)n_chunks, mk, mv, (const bf16*)q,
                       (const bf16*)k_cache, (const bf16*)v_cache, block_table, table_width, seq_past, ws, counters,
                       (bf16*)out, H, G, window, scale * 1.4426950408889634f, n_chunks, cluster_merge);
  else
    launch_pdl(kernel, grid, dim3(DEC_WARPS * 32), smem, stream, mk, mv, (const bf16*)q, (const bf16*)k_cache,
               (const bf16*)v_cache, block_table, table_width, seq_past, ws, counters, (bf16*)out, H, G, window,
               scale * 1.4426950408889634f, n_chunks, cluster_merge);
  return LLMX_LAUNCH_STATUS();
}

// q, out: bf16 [B, H*D] (one token per sequence, in batch order); seq_past[b] = the token's position.
// k_cache, v_cache: one cache entry [n_pages, G, 64, D], 16-byte aligned.
// Every sequence's visible keys are cut into n_chunks <= 32 shares.  With n_chunks > 8: ws is a float32 workspace
// of B*H*n_chunks*(D+4) elements (16-byte aligned), and counters holds B * G * ceil((H/G)/8) words that are zero before the first
// launch (each launch leaves them zero).
LLMX_API int llmx_attention_decode(const void* q, void* out, const void* k_cache, const void* v_cache,
                                   long long n_pages, const int* block_table, int table_width, const int* seq_past, float* ws,
                                   unsigned int* counters, int B, int H, int G, int D, int window, float scale,
                                   int n_chunks, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || window < 0 || n_chunks < 1 || n_chunks > DEC_MAX_CHUNKS ||
      (n_chunks > 8 && (!ws || !counters || ((uintptr_t)ws & 15))) || n_pages <= 0 ||
      ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)q & 3))
    return LLMX_REFUSED(1);
  if (B > 65535 || (long long)G * ((H / G + DEC_ROWS - 1) / DEC_ROWS) > 65535) return LLMX_REFUSED(3);
#define CASE(DD)                                                                                               \
  case DD:                                                                                                     \
    return launch_decode<DD>(q, out, k_cache, v_cache, n_pages, block_table, table_width, seq_past, ws, counters, \
                             B, H, G, window, scale, n_chunks, stream)
  switch (D) {
    CASE(16); CASE(32); CASE(48); CASE(64); CASE(80); CASE(96); CASE(112); CASE(128);
    CASE(144); CASE(160); CASE(176); CASE(192); CASE(208); CASE(224); CASE(240); CASE(256);
    default: return LLMX_REFUSED(1);
  }
#undef CASE
}

// 0; 1 after a launch in which a copy into shared memory never completed, 2 after one whose shared memory was
// not aligned for the swizzled layout (the results are then wrong); reading it clears it.
LLMX_API int llmx_attention_decode_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_dec_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_dec_status, &zero, sizeof(int));
  return v;
}

// ---------------------------------------------------------------------------
// The same kernels for callers that must not allocate: the workspace is a
// file-scope device array.  See attention_decode_noalloc.h for who needs this
// and for the rules (size limit, first call outside capture, shared array).
// ---------------------------------------------------------------------------
#include "attention_decode_noalloc.h"

static __device__ __align__(256) float g_noalloc_workspace[LLMX_NOALLOC_WS_FLOATS];
static __device__ __align__(256) unsigned int g_noalloc_counters[LLMX_NOALLOC_COUNTERS];

// In host code an array's name is only a handle for the runtime, not an address a kernel can use:
// the device addresses are asked for once per device, with that device current, and kept.
#define LLMX_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[LLMX_NOALLOC_MAX_DEVICES];
static unsigned int* g_noalloc_ctr[LLMX_NOALLOC_MAX_DEVICES];

LLMX_API int llmx_attention_decode_noalloc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                           long long n_pages, const int* block_table, int table_width, const int* seq_past, int B,
                                           int H, int G, int D, int window, float scale, int n_chunks,
                                           cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || n_chunks < 1) return LLMX_REFUSED(1);
  // Up to 8 shares merge inside a thread-block cluster and touch neither array: no limit applies to them.
  if (n_chunks > 8) {
    const unsigned long long need = (unsigned long long)B * H * n_chunks * (unsigned long long)DEC_WS_ROW(D);
    const unsigned long long groups = (unsigned long long)B * G * ((H / G + DEC_ROWS - 1) / DEC_ROWS);
    if (need > LLMX_NOALLOC_WS_FLOATS || groups > LLMX_NOALLOC_COUNTERS) return LLMX_NOALLOC_TOO_LARGE;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= LLMX_NOALLOC_MAX_DEVICES) return LLMX_REFUSED(3);
  if (!g_noalloc_ptr[dev] || !g_noalloc_ctr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_workspace);
    if (e != cudaSuccess) return (int)e;
    void* c = nullptr;
    e = cudaGetSymbolAddress(&c, g_noalloc_counters);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_ptr[dev] = static_cast<float*>(p);
    g_noalloc_ctr[dev] = static_cast<unsigned int*>(c);
  }
  return llmx_attention_decode(q, out, k_cache, v_cache, n_pages, block_table, table_width, seq_past, g_noalloc_ptr[dev],
                               g_noalloc_ctr[dev], B, H, G, D, window, scale, n_chunks, stream);
}
