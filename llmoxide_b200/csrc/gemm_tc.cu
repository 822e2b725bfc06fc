// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05) of
// sm_100a:  Y[T,N] = X[T,K] * W[N,K]^T, float32 accumulation in tensor memory.
//
// The weight matrix is the MMA's M operand: a CTA owns 128 rows of W (128
// output features) and a tile of BN tokens, so the same kernel serves decode
// (BN = 16..64 tokens, the weights streamed once at full HBM rate) and prefill
// (BN = 256 tokens).  Both operands are K-major in global memory, so neither
// needs a transpose.  Per CTA:
//   warp 0      producer: TMA (cp.async.bulk.tensor, 128-byte swizzle) loads of
//               the W tile [128 x 64] and the X tile [BN x 64] per stage
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma
//               (M = 128, N = BN, K = 16, four per stage) and commits each
//               stage back to the producer through an mbarrier
//   warps 2..5  epilogue: tcgen05.ld the accumulator (lane = output feature,
//               column = token), convert, store; or store float32 partials
//               of a split reduction; or, with two accumulators (gate and up
//               rows of the same features), silu(gate) * up
// CTAs are persistent: each walks several (row tile, token tile, K split) units
// with the TMA ring running on across units and two accumulator sets in tensor
// memory, so a unit's epilogue overlaps the next unit's MMAs.  Prompt-sized token
// tiles run on CTA pairs (cta_group::2, second kernel below).
// Every wait on an mbarrier is bounded; when one runs out the CTA records it
// in a status word, stops issuing work, frees its tensor memory and returns.
//
// y[t,o] = sum_i W[o,i] x[t,i] (crates/model/src/ops.rs:83-101); the gated
// epilogue is crates/model/src/qwen35/cpu.rs:386-392.
#include "tc_ptx.cuh"

#define TC_BM 128        // rows of W per CTA = MMA M
#define TC_BK 64         // bf16 elements per stage along K = one 128-byte swizzle row
#define TC_UMMA_K 16
#define TC_THREADS 192

__device__ int g_tc_status = 0;   // 0, or which bounded wait ran out: 1 producer, 2 MMA, 3 epilogue, 4 MMA on the accumulator
                                  // (11..14: the same roles of the CTA-pair kernel)
__device__ __forceinline__ void tc_report(int code) {
  atomicExch(&g_tc_status, code);
  llmx_report(code);
}

// Row scales in the epilogue, for a step of few tokens (T <= 64).  The norm before a product may hand over
// x~ = bf16(h * gain) and partial sums of squares of h instead of normalised rows (elementwise.cu,
// add_gain_sumsq): rmsnorm(h) * gain = x~ * r with r[t] = 1 / sqrt(mean(h[t]^2) + eps), and a product is linear
// in its input rows, so r[t] multiplies the accumulator's column t in the epilogue, before any activation
// (crates/model/src/ops.rs:40-59 is the norm).  The partial sums are added in a fixed order.
struct TcScale {
  const float* sumsq;          // [parts][stride]; nullptr: no scaling
  int parts, stride;
  float eps, d;
};

// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t umma_idesc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

// ---------------------------------------------------------------------------
// Epilogue of one accumulator tile: this warp's quarter (32 lanes = 32 rows of
// W) of BN token columns, 16 columns at a time.
// MODE 0: out[t, n] = acc.          MODE 1: two accumulators (gate, up): out[t, n] = silu(gate) * up.
// MODE 2: W's rows come in blocks of 32 = 16 gate rows then the 16 up rows of the same features, so a warp's
//         lanes 0..15 hold gate and lanes 16..31 hold up of the same 16 features: one shuffle per pair of
//         columns brings the two together (the lower lanes finish the even columns, the upper lanes the odd
//         ones), and no warp waits for another.  A tile of 128 rows gives 64 features:
//         out[t, n0/2 + 16 * quad + lane % 16] = silu(gate) * up.
// ---------------------------------------------------------------------------
#define TC_FUSE_BYTES (64 * 4)                    // row scales

template <int BN, int MODE, typename TY>
__device__ __forceinline__ void epilogue_tile(uint32_t acc_addr, bool have_acc, bool store, TY* __restrict__ out,
                                              int n0, int t0, int T, int n_limit, long long ldy, int quad, int lane,
                                              const float* row_scale = nullptr) {
  const int row = quad * 32 + lane;
  const int n = MODE == 2 ? (n0 >> 1) + quad * 16 + (lane & 15) : n0 + row;
  const bool upper = lane >= 16;
#pragma unroll 1
  for (int c = 0; c < BN; c += 16) {
    if (t0 + c >= T) break;
    float v[16], g[16];
    if (have_acc) {
      tmem_ld16(acc_addr + (uint32_t)c, v);
      if (MODE == 1) tmem_ld16(acc_addr + (uint32_t)(BN + c), g);
    } else {
#pragma unroll
      for (int e = 0; e < 16; ++e) v[e] = g[e] = 0.f;
    }
    if (row_scale) {            // column t of the accumulator times r[t] (tokens past T are never stored)
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const float r = row_scale[min(t0 + c + e, 63)];
        v[e] *= r;
        if (MODE == 1) g[e] *= r;
      }
    }
    if (MODE == 2) {
#pragma unroll
      for (int e = 0; e < 16; e += 2) {
        const float got = __shfl_xor_sync(0xffffffffu, upper ? v[e] : v[e + 1], 16);
        const float gate = upper ? got : v[e];
        const float up = upper ? v[e + 1] : got;
        const int t = t0 + c + e + (upper ? 1 : 0);
        if (store && n < n_limit && t < T)
          out[(size_t)t * ldy + n] = from_f32<TY>(__fdividef(gate, 1.0f + __expf(-gate)) * up);
      }
    } else if (store && n < n_limit) {
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const int t = t0 + c + e;
        if (t < T) {
          float r = v[e];
          if (MODE != 0) r = __fdividef(r, 1.0f + __expf(-r)) * g[e];
          out[(size_t)t * ldy + n] = from_f32<TY>(r);
        }
      }
    }
  }
}

// The same tile by way of shared memory, for prompt-sized steps (MODE 0 or 2): the four epilogue warps write
// EP_ROWS tokens x EP_COLS features to one of two staging buffers, token after token as in Y, and one thread
// sends the buffer off as a bulk tensor store.  A warp's direct stores reach only 64 bytes of a token's row each
// (lane = feature), sixteen to a chunk; at 256 tokens a tile they cost four times what the rest of the
// epilogue does, and a kernel's last tile has no MMAs of a next one to hide behind.
template <typename TY>
struct TcStage {
  static constexpr int ROWS = 64 / sizeof(TY);      // tokens per chunk: 32 (bfloat16) or 16 (float32)
};
#define TC_STAGE_BYTES (2 * 32 * 128 * 2)            // two buffers of [ROWS][128 features]

template <int BN, int MODE, typename TY>
__device__ __forceinline__ void epilogue_tile_staged(uint32_t acc_addr, const CUtensorMap* map_y, TY* stage,
                                                     int& chunk_no, int n0, int t0, int split, int T, int quad,
                                                     int lane, bool first_thread, bool accumulate) {
  static_assert(MODE != 1, "one accumulator");
  constexpr int ROWS = TcStage<TY>::ROWS;
  constexpr int COLS = MODE == 2 ? 64 : 128;
  const bool upper = lane >= 16;
  const int col = MODE == 2 ? quad * 16 + (lane & 15) : quad * 32 + lane;
#pragma unroll 1
  for (int c = 0; c < BN; c += ROWS) {
    if (t0 + c >= T) break;
    float v[ROWS];
    if (ROWS == 32) tmem_ld32(acc_addr + (uint32_t)c, v);
    else tmem_ld16(acc_addr + (uint32_t)c, v);
    TY* buf = stage + (size_t)(chunk_no & 1) * ROWS * COLS;
    if (first_thread) bulk_wait_read<1>();              // the store that last read this buffer is done with it
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (MODE == 2) {
#pragma unroll
      for (int e = 0; e < ROWS; e += 2) {
        const float got = __shfl_xor_sync(0xffffffffu, upper ? v[e] : v[e + 1], 16);
        const float gate = upper ? got : v[e];
        const float up = upper ? v[e + 1] : got;
        buf[(e + (upper ? 1 : 0)) * COLS + col] = from_f32<TY>(__fdividef(gate, 1.0f + __expf(-gate)) * up);
      }
    } else {
#pragma unroll
      for (int e = 0; e < ROWS; ++e) buf[e * COLS + col] = from_f32<TY>(v[e]);
    }
    fence_proxy_async();
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (first_thread) {
      if (accumulate) tma_reduce_add_3d(map_y, n0, t0 + c, 0, smem_u32(buf));    // Y += tile (MODE 0, float32)
      else tma_store_3d(map_y, MODE == 2 ? (n0 >> 1) : n0, t0 + c, split, smem_u32(buf));
    }
    ++chunk_no;
  }
}

// ---------------------------------------------------------------------------
// The kernel: persistent CTAs over work units.  A unit is (tile of 128 rows
// of W, tile of BN tokens, one split of K); unit u = ((split * row_tiles +
// row_tile) * token_tiles + token_tile), so CTAs that run side by side share
// a W tile through L2.  CTA c takes units c, c + gridDim.x, ...  The TMA ring
// runs on across unit boundaries, and tensor memory holds two accumulator
// sets, so the epilogue of a unit overlaps the MMAs of the next.
// MODE 0: Y (bf16 or f32) [T, N] or split partials f32 [n_split][T, N].
// MODE 1: two accumulators, rows n and n + F of W; act[T, F] = silu(g) * u.
// ---------------------------------------------------------------------------
template <int BN, int MODE, typename TY>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               TY* __restrict__ Y, int T, int N, int K, long long ldy, int k_blocks_per_split,
               long long split_stride, int F, int n_stages, int row_tiles, int token_tiles, int n_units,
               const TcScale sc) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int N_ACC = MODE == 1 ? 2 : 1;   // MODE 2 has one accumulator: gate and up rows share a tile
  constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;
  constexpr uint32_t B_BYTES = BN * TC_BK * 2;
  constexpr uint32_t STAGE_BYTES = N_ACC * A_BYTES + B_BYTES;
  constexpr uint32_t ACC_COLS = N_ACC * BN;                                  // columns of one accumulator set
  constexpr int ACC_BUFS = (2 * ACC_COLS <= 512) ? 2 : 1;                    // two sets where tensor memory has room
  constexpr uint32_t TMEM_COLS = (ACC_BUFS * ACC_COLS) < 32 ? 32 : (ACC_BUFS * ACC_COLS);   // a power of two >= 32

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_kb = (K + TC_BK - 1) / TC_BK;

  // 1024-byte aligned stage buffers, then the barriers
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + (size_t)n_stages * STAGE_BYTES);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8u * n_stages;
  const uint32_t acc_full0 = empty0 + 8u * n_stages, acc_empty0 = acc_full0 + 16u;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * n_stages + 4);
  float* row_scales = reinterpret_cast<float*>(bars + 2 * n_stages + 6);   // [64] r[t]

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(full0 + 8u * s, 1);
      mbar_init(empty0 + 8u * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full0 + 8u * i, 1);
      mbar_init(acc_empty0 + 8u * i, 4);      // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // unit -> coordinates
  auto unit_coords = [&](int u, int& n0, int& t0, int& kb_begin, int& n_kb, int& split) {
    const int tt = u % token_tiles;
    const int rest = u / token_tiles;
    const int rt = rest % row_tiles;
    split = rest / row_tiles;
    n0 = rt * TC_BM;
    t0 = tt * BN;
    kb_begin = split * k_blocks_per_split;
    const int kb_end = min(total_kb, kb_begin + k_blocks_per_split);
    n_kb = max(0, kb_end - kb_begin);
  };

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      RingPos pos{0, 0};          // where the next k-block goes
      bool waited = false, ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
        int n0, t0, kb_begin, n_kb, split;
        unit_coords(u, n0, t0, kb_begin, n_kb, split);
        int i = 0;
        if (!waited) {
          // The weights do not depend on the kernel before this one: the first stages' weight tiles are
          // requested at once, and only the activation tiles wait for that kernel to finish.
          const int pre = n_kb < n_stages ? n_kb : n_stages;
          for (int j = 0; j < pre; ++j) {
            const uint32_t stage = base + (uint32_t)j * STAGE_BYTES, bar = full0 + 8u * j;
            mbar_expect_tx(bar, STAGE_BYTES);
            const int k = (kb_begin + j) * TC_BK;
            tma_load_2d(stage, &map_w, k, n0, bar);
            if (MODE == 1) tma_load_2d(stage + A_BYTES, &map_w, k, n0 + F, bar);
          }
          pdl_wait();
          waited = true;
          for (int j = 0; j < pre; ++j)
            tma_load_2d(base + (uint32_t)j * STAGE_BYTES + N_ACC * A_BYTES, &map_x, (kb_begin + j) * TC_BK, t0,
                        full0 + 8u * j);
          i = pre;
          if (pre == n_stages) pos = RingPos{0, 1};
          else pos = RingPos{pre, 0};
        }
        for (; i < n_kb; ++i, pos.next(n_stages)) {
          const int s = pos.s;
          if (!mbar_wait(empty0 + 8u * s, pos.phase ^ 1u)) { tc_report(1); ok = false; break; }
          const uint32_t stage = base + (uint32_t)s * STAGE_BYTES;
          const uint32_t bar = full0 + 8u * s;
          mbar_expect_tx(bar, STAGE_BYTES);
          const int k = (kb_begin + i) * TC_BK;
          tma_load_2d(stage, &map_w, k, n0, bar);
          if (MODE == 1) tma_load_2d(stage + A_BYTES, &map_w, k, n0 + F, bar);
          tma_load_2d(stage + N_ACC * A_BYTES, &map_x, k, t0, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BN);
      int j = 0;                  // units done by this CTA
      RingPos pos{0, 0};
      const uint32_t desc0 = umma_desc_lo(base);       // stage 0's W tile; every other tile is an offset from it
      bool ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++j) {
        int n0, t0, kb_begin, n_kb, split;
        unit_coords(u, n0, t0, kb_begin, n_kb, split);
        const int buf = j % ACC_BUFS, use = j / ACC_BUFS;
        const uint32_t acc_addr = tmem_base + (uint32_t)buf * ACC_COLS;
        // the epilogue must have drained this accumulator set (ACC_BUFS units ago)
        if (!mbar_wait(acc_empty0 + 8u * buf, (use & 1) ^ 1)) { tc_report(4); ok = false; break; }
        tc_fence_after();
        for (int i = 0; i < n_kb; ++i, pos.next(n_stages)) {
          const int s = pos.s;
          if (!mbar_wait(full0 + 8u * s, pos.phase)) { tc_report(2); ok = false; break; }
          tc_fence_after();
          const uint32_t da = desc0 + (uint32_t)s * (STAGE_BYTES >> 4);
#pragma unroll
          for (int kk = 0; kk < TC_BK / TC_UMMA_K; ++kk) {
            const uint32_t db = da + ((N_ACC * A_BYTES) >> 4) + kk * ((TC_UMMA_K * 2) >> 4);
            const uint32_t acc = (i > 0 || kk > 0) ? 1u : 0u;
            umma_bf16_lo(acc_addr, da + kk * ((TC_UMMA_K * 2) >> 4), db, idesc, acc);
            if (MODE == 1)
              umma_bf16_lo(acc_addr + BN, da + (A_BYTES >> 4) + kk * ((TC_UMMA_K * 2) >> 4), db, idesc, acc);
          }
          umma_commit(empty0 + 8u * s);   // the stage is free once these MMAs have read it
        }
        // (tests: with llmx_withhold the first unit's accumulator is never announced, and the epilogue's wait runs out)
        if (!(j == 0 && llmx_withhold))
          umma_commit(acc_full0 + 8u * buf);  // this unit's accumulator is complete once every MMA has finished
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int quad = warp & 3;          // the quarter of tensor memory this warp may read
    const int n_limit = MODE == 0 ? N : F;
    bool waited = false, failed = false;
    const float* row_scale = nullptr;
    if (sc.sumsq) {
      // r[t] for the step's tokens (T <= 64): the partial sums of squares come from the kernel before
      pdl_wait();
      waited = true;
      // one thread per token: its partial sums are loaded together (one trip to L2 for the whole tile; a loop
      // over tokens would make one trip per token and, at 64 tokens, outlast the MMAs) and added in the order
      // of the parts
      const int t = (int)threadIdx.x - 64;
      if (t < T && t < 64) {
        float a = 0.f;
#pragma unroll 8
        for (int p = 0; p < sc.parts; ++p) a += __ldcg(sc.sumsq + (size_t)p * sc.stride + t);
        row_scales[t] = 1.0f / sqrtf(a / sc.d + sc.eps);
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      row_scale = row_scales;
    }
    int j = 0;
    for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++j) {
      int n0, t0, kb_begin, n_kb, split;
      unit_coords(u, n0, t0, kb_begin, n_kb, split);
      const int buf = j % ACC_BUFS, use = j / ACC_BUFS;
      if (!failed) {
        bool ok = mbar_wait(acc_full0 + 8u * buf, use & 1);
        if (!ok && lane == 0) tc_report(3);
        failed = __shfl_sync(0xffffffffu, ok ? 0 : 1, 0) != 0;
      }
      if (failed) break;
      tc_fence_after();
      if (n_kb == 0 && !waited) {       // no load ordered this unit after the kernel before: do it here
        pdl_wait();
        waited = true;
      }
      TY* out = Y + (MODE == 0 ? (size_t)split * split_stride : 0);
      const uint32_t acc_addr = tmem_base + (uint32_t)buf * ACC_COLS + ((uint32_t)(quad * 32) << 16);
      epilogue_tile<BN, MODE, TY>(acc_addr, n_kb > 0, true, out, n0, t0, T, n_limit, ldy, quad, lane, row_scale);
      // hand the accumulator set back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8u * buf) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
  if (threadIdx.x == 0) LLMX_MARK(21);      // (timeline builds only: when this CTA was done)
}

// ---------------------------------------------------------------------------
// The same product on CTA pairs (tcgen05 cta_group::2) for prompt-sized token
// tiles.  A cluster of two CTAs on neighbouring SMs owns 256 rows of W and a
// tile of BN tokens: each CTA loads its own 128 rows of W and HALF of the
// token tile, and the leader CTA issues one MMA of M = 256, N = BN that reads
// both CTAs' shared memory and writes both CTAs' tensor memory.  Per SM that is
// 32 KB of operands per 512 MMA cycles instead of 48 KB, which is what the
// single-CTA kernel starves on.  Barriers: the leader's `full` barrier counts
// one expect-tx arrival from each CTA's producer (TMA with cta_group::2 may
// signal the peer's barrier); `empty` and `acc_full` are signalled in both
// CTAs by one multicast tcgen05.commit; both CTAs' epilogue warps arrive on
// the leader's `acc_empty`.  Every wait is bounded.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64(), limit = llmx_wait_cycles;
  while (!mbar_try_wait_cluster(bar, parity)) {
    if (clock64() - t0 > limit) return false;
  }
  return true;
}
__device__ __forceinline__ void mbar_remote_expect_tx(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair_lo(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\n.reg .b64 da, db;\n"
      "mov.b64 da, {%1, %5};\nmov.b64 db, {%2, %5};\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %3, p;\n}"
      ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(UMMA_DESC_HI)
      : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {   // arrives on `bar` in both CTAs
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3)
      : "memory");
}
__host__ __device__ constexpr uint32_t umma_idesc_pair(int n) {   // M = 256 over the pair
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

// Units: (pair of row tiles = 256 rows of W, tile of BN tokens).  Token tiles come in groups of `group_tiles`;
// a group's units run token tile fastest, then row pair, and group follows group.  The pairs that run side by
// side then share a few W tiles through L2, and a group's activations (chosen by the host to fit well inside
// L2) are fetched from memory once and serve every row pair, however many tokens the step has; W is streamed
// once per group.  With one group this is "token tile fastest" over the whole product.  A short prompt against a
// narrow matrix has fewer units than the GPU has pairs; its reduction is then split (the units of split 0, then
// those of split 1, ...), each split writing float32 partials of its own for the kernel that consumes them.
template <int BN, int MODE, typename TY>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const __grid_constant__ CUtensorMap map_y, TY* __restrict__ Y, int T, int N, int K, long long ldy,
                    int F, int n_stages, int row_pairs, int token_tiles, int n_units, int group_tiles, int staged,
                    int accumulate, int kb_per_split, long long split_stride) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int N_ACC = MODE == 1 ? 2 : 1;
  constexpr int HALF = BN / 2;                                              // tokens this CTA loads
  constexpr uint32_t A_BYTES = TC_BM * TC_BK * 2;
  constexpr uint32_t B_BYTES = HALF * TC_BK * 2;
  constexpr uint32_t STAGE_BYTES = N_ACC * A_BYTES + B_BYTES;                // per CTA
  constexpr uint32_t ACC_COLS = N_ACC * BN;
  constexpr int ACC_BUFS = (2 * ACC_COLS <= 512) ? 2 : 1;
  constexpr uint32_t TMEM_COLS = ACC_BUFS * ACC_COLS;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int total_kb = (K + TC_BK - 1) / TC_BK;

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + (size_t)n_stages * STAGE_BYTES);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8u * n_stages;
  const uint32_t acc_full0 = empty0 + 8u * n_stages, acc_empty0 = acc_full0 + 16u;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * n_stages + 4);
  volatile uint32_t* epi_failed = reinterpret_cast<volatile uint32_t*>(bars + 2 * n_stages + 5);
  TY* stage_buf = reinterpret_cast<TY*>(base_ptr + (size_t)n_stages * STAGE_BYTES + 256);   // after the barriers
  // the leader's copies of the barriers that both CTAs signal
  const uint32_t leader_full0 = map_to_cta(full0, 0), leader_acc_empty0 = map_to_cta(acc_empty0, 0);

  pdl_launch_dependents();
  // Rule: a CTA pair waits for the kernel before it ahead of any set-up.  Its tensor-memory allocation for the
  // pair, its cluster barrier and its first weight tiles must not be in progress while CTAs of the kernel before
  // still hold tensor memory and shared memory on the same SMs: two kernels each waiting for what the other
  // holds do not finish.  Prompt-sized products lose next to nothing: the set-up is microseconds against hundreds.
  pdl_wait();
  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(full0 + 8u * s, 2);        // one expect-tx arrival per CTA (used in the leader only)
      mbar_init(empty0 + 8u * s, 1);       // the multicast commit
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full0 + 8u * i, 1);    // the multicast commit
      mbar_init(acc_empty0 + 8u * i, 8);   // four epilogue warps of each CTA (used in the leader only)
    }
    *epi_failed = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    if (staged) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_y) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();                      // barriers and tensor memory of both CTAs are ready
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  auto unit_coords = [&](int u, int& n0, int& t0, int& split, int& kb_begin, int& n_kb) {
    const int per_split = row_pairs * token_tiles;
    split = u / per_split;
    u -= split * per_split;
    kb_begin = split * kb_per_split;
    n_kb = min(total_kb, kb_begin + kb_per_split) - kb_begin;          // (the host leaves no split empty)
    const int per_group = group_tiles * row_pairs;
    const int g = u / per_group, r = u - g * per_group;
    const int here = min(group_tiles, token_tiles - g * group_tiles);     // the last group may be narrower
    const int rp = r / here, tt = g * group_tiles + (r - rp * here);
    n0 = rp * 2 * TC_BM + (int)rank * TC_BM;                  // this CTA's 128 rows
    t0 = tt * BN;
  };

  if (warp == 0) {
    // ---------------- producer (one per CTA) ----------------
    if (lane == 0) {
      RingPos pos{0, 0};
      bool waited = false, ok = true;
      for (int u = pair; u < n_units && ok; u += n_pairs) {
        int n0, t0, split, kb_begin, n_kb;
        unit_coords(u, n0, t0, split, kb_begin, n_kb);
        const int tx = t0 + (int)rank * HALF;                 // this CTA's half of the token tile
        int i = 0;
        if (!waited) {
          const int pre = n_kb < n_stages ? n_kb : n_stages;
          for (int j = 0; j < pre; ++j) {
            const uint32_t stage = base + (uint32_t)j * STAGE_BYTES, bar = leader_full0 + 8u * j;
            mbar_remote_expect_tx(bar, STAGE_BYTES);
            tma_load_2d_pair(stage, &map_w, (kb_begin + j) * TC_BK, n0, bar);
            if (MODE == 1) tma_load_2d_pair(stage + A_BYTES, &map_w, (kb_begin + j) * TC_BK, n0 + F, bar);
          }
          waited = true;                    // (the CTA waited for the kernel before it at its start)
          for (int j = 0; j < pre; ++j)
            tma_load_2d_pair(base + (uint32_t)j * STAGE_BYTES + N_ACC * A_BYTES, &map_x, (kb_begin + j) * TC_BK, tx,
                             leader_full0 + 8u * j);
          i = pre;
          if (pre == n_stages) pos = RingPos{0, 1};
          else pos = RingPos{pre, 0};
        }
        for (; i < n_kb; ++i, pos.next(n_stages)) {
          const int s = pos.s;
          if (!mbar_wait_cluster(empty0 + 8u * s, pos.phase ^ 1u)) { tc_report(11); ok = false; break; }
          const uint32_t stage = base + (uint32_t)s * STAGE_BYTES, bar = leader_full0 + 8u * s;
          mbar_remote_expect_tx(bar, STAGE_BYTES);
          const int k = (kb_begin + i) * TC_BK;
          tma_load_2d_pair(stage, &map_w, k, n0, bar);
          if (MODE == 1) tma_load_2d_pair(stage + A_BYTES, &map_w, k, n0 + F, bar);
          tma_load_2d_pair(stage + N_ACC * A_BYTES, &map_x, k, tx, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_pair(BN);
      int j = 0;
      RingPos pos{0, 0};
      const uint32_t desc0 = umma_desc_lo(base);       // stage 0's W tile; every other tile is an offset from it
      bool ok = true;
      for (int u = pair; u < n_units && ok; u += n_pairs, ++j) {
        int n0, t0, split, kb_begin, n_kb;
        unit_coords(u, n0, t0, split, kb_begin, n_kb);
        const int buf = j % ACC_BUFS, use = j / ACC_BUFS;
        const uint32_t acc_addr = tmem_base + (uint32_t)buf * ACC_COLS;
        if (!mbar_wait_cluster(acc_empty0 + 8u * buf, (use & 1) ^ 1)) { tc_report(14); ok = false; break; }
        tc_fence_after();
        for (int i = 0; i < n_kb; ++i, pos.next(n_stages)) {
          const int s = pos.s;
          if (!mbar_wait_cluster(full0 + 8u * s, pos.phase)) { tc_report(12); ok = false; break; }
          tc_fence_after();
          const uint32_t da = desc0 + (uint32_t)s * (STAGE_BYTES >> 4);
#pragma unroll
          for (int kk = 0; kk < TC_BK / TC_UMMA_K; ++kk) {
            const uint32_t db = da + ((N_ACC * A_BYTES) >> 4) + kk * ((TC_UMMA_K * 2) >> 4);
            const uint32_t acc = (i > 0 || kk > 0) ? 1u : 0u;
            umma_bf16_pair_lo(acc_addr, da + kk * ((TC_UMMA_K * 2) >> 4), db, idesc, acc);
            if (MODE == 1)
              umma_bf16_pair_lo(acc_addr + BN, da + (A_BYTES >> 4) + kk * ((TC_UMMA_K * 2) >> 4), db, idesc, acc);
          }
          umma_commit_pair(empty0 + 8u * s);
        }
        if (!(j == 0 && llmx_withhold))     // (tests: the first unit's accumulator is never announced)
          umma_commit_pair(acc_full0 + 8u * buf);
      }
    }
  } else {
    // ---------------- epilogue (both CTAs) ----------------
    const int quad = warp & 3;
    const int n_limit = MODE == 0 ? N : F;
    bool failed = false;
    int j = 0, chunk_no = 0;
    for (int u = pair; u < n_units; u += n_pairs, ++j) {
      int n0, t0, split, kb_begin, n_kb;
      unit_coords(u, n0, t0, split, kb_begin, n_kb);
      const int buf = j % ACC_BUFS, use = j / ACC_BUFS;
      if (!failed) {
        bool ok = mbar_wait_cluster(acc_full0 + 8u * buf, use & 1);
        if (!ok && lane == 0) tc_report(13);
        failed = __shfl_sync(0xffffffffu, ok ? 0 : 1, 0) != 0;
      }
      if (MODE != 1 && staged) {
        // the four warps meet at barriers inside the staged epilogue, so they leave together or not at all
        if (failed && lane == 0) *epi_failed = 1u;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        failed = *epi_failed != 0u;
      }
      if (failed) break;
      tc_fence_after();
      const uint32_t acc_addr = tmem_base + (uint32_t)buf * ACC_COLS + ((uint32_t)(quad * 32) << 16);
      if (MODE != 1 && staged)
        epilogue_tile_staged<BN, MODE == 1 ? 0 : MODE, TY>(acc_addr, &map_y, stage_buf, chunk_no, n0, t0, split, T, quad,
                                                             lane, threadIdx.x == 64, accumulate != 0);
      else
        epilogue_tile<BN, MODE, TY>(acc_addr, true, true, Y + (size_t)split * split_stride, n0, t0, T, n_limit, ldy, quad,
                                    lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_remote_arrive(leader_acc_empty0 + 8u * buf);
    }
    if (threadIdx.x == 64) bulk_wait_all();    // this CTA's stores are in global memory before it ends
  }
  tc_fence_before();
  cluster_sync_all();                      // the peer may still read this CTA's shared and tensor memory until here
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

template <int BN, int MODE, typename TY>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, void* Y, int T, int N, int K, long long ldy,
                  int n_split, long long split_stride, int F, const TcScale& sc, cudaStream_t stream) {
  constexpr int N_ACC = MODE == 1 ? 2 : 1;
  constexpr size_t STAGE = (size_t)N_ACC * TC_BM * TC_BK * 2 + (size_t)BN * TC_BK * 2;
  const int total_kb = (K + TC_BK - 1) / TC_BK;
  const int per_split = (total_kb + n_split - 1) / n_split;
  const int rows = MODE == 1 ? F : N;   // MODE 2 walks all 2F interleaved rows
  const int row_tiles = (rows + TC_BM - 1) / TC_BM, token_tiles = (T + BN - 1) / BN;
  const long long n_units = (long long)row_tiles * token_tiles * n_split;
  if (n_units > 0x7fffffff) return LLMX_REFUSED(3);
  // Decode tiles (few tokens) stream weights: two CTAs per SM, so that more loads are in flight per SM.
  // 128-token tiles do the same when there are more units than SMs (gate|up: 192 units are then resident at
  // once instead of running a second round on a third of the SMs; two accumulator sets of 128 columns per
  // CTA, so the two CTAs fill tensor memory; not MODE 1, whose CTA takes all of it); with a CTA per SM or
  // fewer they keep the deep ring.  Wider tiles take the whole SM.
  const int ctas_per_sm = BN <= 64 || (BN == 128 && MODE != 1 && n_units > sm_count()) ? 2 : 1;
  // (108 KB: six stages of a 16-token tile, three of a 128-token tile; two such CTAs and the driver's 1 KB
  // each still fit the SM's 228 KB)
  const size_t budget = ctas_per_sm == 2 ? 108 * 1024 : 200 * 1024;
  int stages = (int)(budget / STAGE);
  if (stages > 12) stages = 12;
  if (stages < 2) stages = 2;
  const size_t smem = 1024 + (size_t)stages * STAGE + (2 * stages + 6) * 8 +
                      TC_FUSE_BYTES;
  auto kernel = gemm_tc_kernel<BN, MODE, TY>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int max_ctas = sm_count() * ctas_per_sm;
  const int grid = n_units < max_ctas ? (int)n_units : max_ctas;
  launch_pdl(kernel, dim3(grid), dim3(TC_THREADS), smem, stream, mw, mx, (TY*)Y, T, N, K, ldy, per_split,
             split_stride, F, stages, row_tiles, token_tiles, (int)n_units, sc);
  return LLMX_LAUNCH_STATUS();
}

// X [T,K] bf16 (row stride ldx), W [N,K] bf16 (row stride ldw).
// mode 0: Y [T,N] of y_dtype, or with n_split > 1 float32 partials [n_split][T,N] (split_stride elements apart).
// mode 1: W = [gate rows; up rows] with N = 2F; Y = act [T,F] of y_dtype.
// mode 2: W = blocks of 32 rows, each 16 gate rows then the 16 up rows of the same features (N = 2F, F % 16 == 0);
//         Y = act [T,F] bf16.
// The same with row scales applied in the epilogue (see TcScale): in_sumsq [in_parts][in_stride >= T], T <= 64.
LLMX_API int llmx_gemm_tc_scaled(const void* X, const void* W, void* Y, int y_dtype, int T, int N, int K, long long ldx,
                                 long long ldw, long long ldy, int n_split, long long split_stride, int mode,
                                 const float* in_sumsq, int in_parts, int in_stride, float in_eps, int in_d,
                                 cudaStream_t stream);

LLMX_API int llmx_gemm_tc(const void* X, const void* W, void* Y, int y_dtype, int T, int N, int K, long long ldx,
                          long long ldw, long long ldy, int n_split, long long split_stride, int mode,
                          cudaStream_t stream) {
  return llmx_gemm_tc_scaled(X, W, Y, y_dtype, T, N, K, ldx, ldw, ldy, n_split, split_stride, mode, nullptr, 0, 0, 0.f,
                             1, stream);
}

LLMX_API int llmx_gemm_tc_scaled(const void* X, const void* W, void* Y, int y_dtype, int T, int N, int K, long long ldx,
                                 long long ldw, long long ldy, int n_split, long long split_stride, int mode,
                                 const float* in_sumsq, int in_parts, int in_stride, float in_eps, int in_d,
                                 cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  TcScale sc = {};
  if (in_sumsq) {
    if (T > 64 || in_parts <= 0 || in_stride < T || in_d <= 0) return LLMX_REFUSED(1);
    sc.sumsq = in_sumsq, sc.parts = in_parts, sc.stride = in_stride, sc.eps = in_eps, sc.d = (float)in_d;
  }
  if (K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return LLMX_REFUSED(1);
  if (n_split < 1 || (n_split > 1 && (mode != 0 || y_dtype != LLMX_F32))) return LLMX_REFUSED(1);
  if (mode < 0 || mode > 2 || (mode == 1 && (N % 2)) || (mode == 2 && (N % 32))) return LLMX_REFUSED(1);
  const int F = mode != 0 ? N / 2 : 0;
  int bn = 16;
  while (bn < T && bn < (mode == 1 ? 128 : 256)) bn <<= 1;
  CUtensorMap mw, mx;
  if (make_map(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, TC_BM, true)) return LLMX_REFUSED(4);
  if (make_map(&mx, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, (uint32_t)bn, false)) return LLMX_REFUSED(4);
#define GO(BN, MODE, TY) return launch<BN, MODE, TY>(mw, mx, Y, T, N, K, ldy, n_split, split_stride, F, sc, stream)
#define BY_BN(MODE, TY)                    \
  switch (bn) {                            \
    case 16: GO(16, MODE, TY);             \
    case 32: GO(32, MODE, TY);             \
    case 64: GO(64, MODE, TY);             \
    case 128: GO(128, MODE, TY);           \
    default: GO(256, MODE, TY);            \
  }
  if (mode == 0 && y_dtype == LLMX_BF16) { BY_BN(0, bf16) }
  if (mode == 0 && y_dtype == LLMX_F32) { BY_BN(0, float) }
  if (mode == 1 && y_dtype == LLMX_BF16) {
    switch (bn) {
      case 16: GO(16, 1, bf16);
      case 32: GO(32, 1, bf16);
      case 64: GO(64, 1, bf16);
      case 128: GO(128, 1, bf16);
      default: GO(256, 1, bf16);
    }
  }
  if (mode == 2 && y_dtype == LLMX_BF16) { BY_BN(2, bf16) }
#undef BY_BN
#undef GO
  return LLMX_REFUSED(2);
}

template <int BN, int MODE, typename TY>
static int launch_pair(const CUtensorMap& mw, const CUtensorMap& mx, void* Y, int T, int N, int K, long long ldy,
                       int F, int accumulate, int n_split, long long split_stride, cudaStream_t stream) {
  constexpr int N_ACC = MODE == 1 ? 2 : 1;
  constexpr size_t STAGE = (size_t)N_ACC * TC_BM * TC_BK * 2 + (size_t)(BN / 2) * TC_BK * 2;
  int stages = (int)((200 * 1024) / STAGE);
  if (stages > 12) stages = 12;
  // the output tiles leave through a staging buffer and bulk tensor stores where Y allows it
  CUtensorMap my = mw;
  int staged = 0;
  if (MODE != 1 && !((uintptr_t)Y & 15) && !((ldy * (long long)sizeof(TY)) & 15))
    staged = (n_split == 1 || !((split_stride * (long long)sizeof(TY)) & 15)) &&
             make_store_map(&my, Y, (int)sizeof(TY), (uint64_t)n_split, (uint64_t)T, (uint64_t)(MODE == 2 ? F : N),
                            (uint64_t)ldy, (uint64_t)split_stride, TcStage<TY>::ROWS, MODE == 2 ? 64 : 128) == 0;
  if (accumulate && !staged) return LLMX_REFUSED(4);      // Y += ... exists only as a bulk tensor reduction
  const size_t smem = 1024 + (size_t)stages * STAGE + 256 + (MODE != 1 ? TC_STAGE_BYTES : 0);
  auto kernel = gemm_tc_pair_kernel<BN, MODE, TY>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int rows = MODE == 1 ? F : N;
  const int row_pairs = (rows + 2 * TC_BM - 1) / (2 * TC_BM), token_tiles = (T + BN - 1) / BN;
  const int total_kb = (K + TC_BK - 1) / TC_BK;
  const int kb_per_split = (total_kb + n_split - 1) / n_split;
  if ((long long)kb_per_split * (n_split - 1) >= total_kb) return LLMX_REFUSED(1);      // a split without any K
  const long long n_units = (long long)row_pairs * token_tiles * n_split;
  if (n_units > 0x7fffffff) return LLMX_REFUSED(3);
  // token tiles per group: a group's activations (BN tokens x K each) take at most half of L2, and the groups
  // are of about equal size
  static int l2_bytes = 0;
  if (!l2_bytes) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&l2_bytes, cudaDevAttrL2CacheSize, dev) != cudaSuccess || l2_bytes <= 0) l2_bytes = 64 << 20;
  }
  long long most = (l2_bytes / 2) / ((long long)BN * K * 2);
  if (most < 2) most = 2;
  const long long n_groups = (token_tiles + most - 1) / most;
  const long long group_tiles = (token_tiles + n_groups - 1) / n_groups;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = llmx_pdl_allowed();
  cfg.attrs = attr;
  // A persistent grid must fit the GPU at once: not every SM can be half of a pair (it depends on how
  // the SMs are grouped), so the number of pairs that run together is asked for, once per kernel.
  static int max_pairs = 0;
  if (!max_pairs) {
    cfg.gridDim = dim3(sm_count() / 2 * 2);
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) n = sm_count() / 2 - 4;
    max_pairs = n;
  }
  // As many pairs as make the rounds even: 128 units on 74 pairs are two rounds, and two rounds are 64 pairs at
  // work all the time (the step runs at the power cap: ten idle-waiting pairs fewer leave the others more clock).
  const long long rounds = (n_units + max_pairs - 1) / max_pairs;
  const int pairs = (int)((n_units + rounds - 1) / rounds);
  cfg.gridDim = dim3(2 * pairs);
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, mw, mx, my, (TY*)Y, T, N, K, ldy, F, stages, row_pairs, token_tiles,
                                     (int)n_units, (int)group_tiles, staged, accumulate, kb_per_split, split_stride);
  if (e != cudaSuccess) return (int)e;
  return LLMX_LAUNCH_STATUS();
}

// The CTA-pair kernel: prompt-sized token counts only (T > 128).  Same arguments as llmx_gemm_tc (n_split > 1:
// float32 partials [n_split][T,N], split_stride elements apart, mode 0), and
// `accumulate`: Y += X W^T instead of Y = X W^T (mode 0 and float32 Y only: every element receives one
// float32 addition, so the result does not depend on the order in which the tiles arrive).
LLMX_API int llmx_gemm_tc_pair(const void* X, const void* W, void* Y, int y_dtype, int T, int N, int K,
                               long long ldx, long long ldw, long long ldy, int mode, int accumulate, int n_split,
                               long long split_stride, cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return LLMX_REFUSED(1);
  if (T <= 128 || mode < 0 || mode > 2 || (mode == 1 && (N % 2)) || (mode == 2 && (N % 32))) return LLMX_REFUSED(1);
  const int F = mode != 0 ? N / 2 : 0;
  const int bn = mode == 1 ? 128 : 256;
  CUtensorMap mw, mx;
  if (make_map(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, TC_BM, true)) return LLMX_REFUSED(4);
  if (make_map(&mx, X, (uint64_t)T, (uint64_t)K, (uint64_t)ldx, (uint32_t)(bn / 2), false)) return LLMX_REFUSED(4);
  if (accumulate && (mode != 0 || y_dtype != LLMX_F32 || n_split != 1)) return LLMX_REFUSED(1);
  if (n_split < 1 || (n_split > 1 && (mode != 0 || y_dtype != LLMX_F32))) return LLMX_REFUSED(1);
  if (mode == 0 && y_dtype == LLMX_BF16) return launch_pair<256, 0, bf16>(mw, mx, Y, T, N, K, ldy, F, 0, 1, 0, stream);
  if (mode == 0 && y_dtype == LLMX_F32)
    return launch_pair<256, 0, float>(mw, mx, Y, T, N, K, ldy, F, accumulate, n_split, split_stride, stream);
  if (mode == 1 && y_dtype == LLMX_BF16) return launch_pair<128, 1, bf16>(mw, mx, Y, T, N, K, ldy, F, 0, 1, 0, stream);
  if (mode == 2 && y_dtype == LLMX_BF16) return launch_pair<256, 2, bf16>(mw, mx, Y, T, N, K, ldy, F, 0, 1, 0, stream);
  return LLMX_REFUSED(2);
}

// The status word of the bounded waits: 0, or which role gave up.  Reading it synchronises the device.
LLMX_API int llmx_gemm_tc_status(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v) {
    int z = 0;
    cudaMemcpyToSymbol(g_tc_status, &z, sizeof(int));
  }
  return v;
}
