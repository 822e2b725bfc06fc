// Prompt attention over the paged bfloat16 cache: variable-length batches,
// causal, grouped-query, a window or none, whole prompts or later chunks of a
// prompt (queries at positions past..past+T-1 read the cached keys before
// them too).  Tiled online-softmax attention: a CTA owns 64 consecutive query
// tokens of one head and walks the visible keys one cache page (64 keys) at a
// time; scores and the weighted sum run on the tensor cores
// (mma.sync.m16n8k16, bf16 in, f32 out), softmax statistics stay in float32.
//
// Formulas as in attention.cu (crates/model/src/qwen35/cpu.rs:325-355,
// crates/model/src/cache.rs:31-37).  The keys and values of the whole step
// are in the cache before this kernel runs (cpu.rs:314-323).
//
// Shared memory holds the query tile and two stages of (K page, V page),
// filled by cp.async in 16-byte chunks whose position in a row is XORed with
// the row number so that ldmatrix reads are free of bank conflicts.
#include "common.cuh"

#define PF_BQ 64          // query tokens per CTA (4 warps x 16 rows)
#define PF_BK LLMX_PAGE   // keys per tile = one cache page
#define PF_THREADS 128

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

// Byte offset of 16-byte chunk `c` of row `r` in a swizzled tile whose rows hold D bf16.
template <int D>
__device__ __forceinline__ uint32_t swz(int r, int c) {
  return (uint32_t)(r * (D * 2) + ((c ^ (r & 7)) << 4));
}

template <int D>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ k_cache,
                         const bf16* __restrict__ v_cache, const int* __restrict__ block_table, int table_width,
                         const int* __restrict__ seq_start, const int* __restrict__ seq_past, int H, int G,
                         int window, float scale_log2) {
  constexpr int CHUNKS = D / 8;              // 16-byte chunks per row
  constexpr int KSTEPS = D / 16;             // k-steps of the score product
  constexpr int TILE_BYTES = PF_BK * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = (uint32_t)__cvta_generic_to_shared(smem);
  const uint32_t sKV = sQ + PF_BQ * D * 2;   // stage s: K at sKV + s*2*TILE_BYTES, V after it

  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // heads fastest in launch order, query tiles from the last (longest) down: the tail is made of short tiles
  const int b = blockIdx.z, hq = blockIdx.x;
  const int g = hq / (H / G);
  const int tok0 = seq_start[b], n_new = seq_start[b + 1] - tok0;
  const int i0 = (gridDim.y - 1 - blockIdx.y) * PF_BQ;
  if (i0 >= n_new) return;
  const int past = seq_past[b];
  const int rows_here = min(PF_BQ, n_new - i0);
  const int pos_lo = past + i0, pos_hi = past + i0 + rows_here - 1;   // positions of the tile's queries
  const int first_lo = (window > 0 && pos_lo - (window - 1) > 0) ? pos_lo - (window - 1) : 0;
  const int page_first = first_lo / PF_BK, page_last = pos_hi / PF_BK;
  const int n_tiles = page_last - page_first + 1;
  const int* pages = block_table + (size_t)b * table_width;

  // ---- stage the query tile -------------------------------------------------------
  for (int idx = tid; idx < PF_BQ * CHUNKS; idx += PF_THREADS) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const int rr = r < rows_here ? r : rows_here - 1;              // rows past the end repeat the last one
    cp_async16(sQ + swz<D>(r, c), q + ((size_t)(tok0 + i0 + rr) * H + hq) * D + c * 8);
  }
  auto load_tile = [&](int t, int stage) {
    const int phys = pages[page_first + t];
    const bf16* kp = k_cache + cache_row_offset(phys, g, 0, G, D);
    const bf16* vp = v_cache + cache_row_offset(phys, g, 0, G, D);
    const uint32_t sK = sKV + stage * 2 * TILE_BYTES, sV = sK + TILE_BYTES;
    for (int idx = tid; idx < PF_BK * CHUNKS; idx += PF_THREADS) {
      const int r = idx / CHUNKS, c = idx % CHUNKS;
      cp_async16(sK + swz<D>(r, c), kp + (size_t)r * D + c * 8);
      cp_async16(sV + swz<D>(r, c), vp + (size_t)r * D + c * 8);
    }
  };
  load_tile(0, 0);
  cp_async_commit();

  // accumulators: this warp's 16 query rows; a thread holds rows (lane/4) and (lane/4 + 8)
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  uint32_t qf[KSTEPS][4];

  const int row0 = warp * 16 + (lane >> 2);
  const int p0 = past + i0 + row0, p1 = p0 + 8;                    // positions of this thread's two rows
  const int f0 = (window > 0 && p0 - (window - 1) > 0) ? p0 - (window - 1) : 0;
  const int f1 = (window > 0 && p1 - (window - 1) > 0) ? p1 - (window - 1) : 0;

  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t & 1;
    if (t + 1 < n_tiles) {
      load_tile(t + 1, stage ^ 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (t == 0) {
      // query fragments: ldmatrix x4 = rows (lane%16) of the warp's 16, chunks 2*ks + lane/16
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks)
        ldmatrix_x4(sQ + swz<D>(warp * 16 + (lane & 15), 2 * ks + (lane >> 4)), qf[ks][0], qf[ks][1], qf[ks][2],
                    qf[ks][3]);
    }
    const uint32_t sK = sKV + stage * 2 * TILE_BYTES, sV = sK + TILE_BYTES;
    const int key0 = (page_first + t) * PF_BK;
    if (key0 + PF_BK - 1 > pos_hi) {
      // Rows of the page past the sequence's last key were never written (or belong to an earlier owner
      // of the page).  Their weights are exactly 0, but 0 * NaN is NaN, so the values are cleared.
      const int valid = pos_hi - key0 + 1;
      uint8_t* vtile = smem + (sV - sQ);
      for (int idx = tid; idx < (PF_BK - valid) * CHUNKS; idx += PF_THREADS) {
        const int r = valid + idx / CHUNKS, c = idx % CHUNKS;
        *reinterpret_cast<uint4*>(vtile + swz<D>(r, c)) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncthreads();
    }

    // ---- S = Q K^T: 16 x 64 per warp -----------------------------------------------
    float s[PF_BK / 8][4];
#pragma unroll
    for (int j = 0; j < PF_BK / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int jp = 0; jp < PF_BK / 16; ++jp) {
        // one x4 covers keys 16*jp..+15 and dims 16*ks..+15: matrices (keys 0-7, d lo), (keys 0-7, d hi),
        // (keys 8-15, d lo), (keys 8-15, d hi)
        uint32_t b0, b1, b2, b3;
        const int kr = jp * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int kc = 2 * ks + ((lane >> 3) & 1);
        ldmatrix_x4(sK + swz<D>(kr, kc), b0, b1, b2, b3);
        mma_bf16(s[2 * jp], qf[ks], b0, b1);
        mma_bf16(s[2 * jp + 1], qf[ks], b2, b3);
      }
    }

    // ---- mask, running maximum, probabilities -----------------------------------------
    float mx0 = m0, mx1 = m1;
#pragma unroll
    for (int j = 0; j < PF_BK / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = key0 + 8 * j + 2 * (lane & 3) + e;
        s[j][e] = (key >= f0 && key <= p0) ? s[j][e] * scale_log2 : -INFINITY;
        s[j][2 + e] = (key >= f1 && key <= p1) ? s[j][2 + e] * scale_log2 : -INFINITY;
        mx0 = fmaxf(mx0, s[j][e]);
        mx1 = fmaxf(mx1, s[j][2 + e]);
      }
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float ref0 = mx0 == -INFINITY ? 0.f : mx0, ref1 = mx1 == -INFINITY ? 0.f : mx1;
    const float c0 = exp2f(m0 - ref0), c1 = exp2f(m1 - ref1);     // m = -inf gives 0
    m0 = mx0;
    m1 = mx1;
    float sum0 = 0.f, sum1 = 0.f;
    uint32_t pf[PF_BK / 16][4];
#pragma unroll
    for (int j = 0; j < PF_BK / 8; ++j) {
      const float e0 = exp2f(s[j][0] - ref0), e1 = exp2f(s[j][1] - ref0);
      const float e2 = exp2f(s[j][2] - ref1), e3 = exp2f(s[j][3] - ref1);
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

    // ---- O += P V ---------------------------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < PF_BK / 16; ++kk) {
#pragma unroll
      for (int jp = 0; jp < D / 16; ++jp) {
        // transposed x4: matrices (keys 0-7, d lo), (keys 8-15, d lo), (keys 0-7, d hi), (keys 8-15, d hi)
        uint32_t b0, b1, b2, b3;
        const int vr = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int vc = 2 * jp + (lane >> 4);
        ldmatrix_x4_trans(sV + swz<D>(vr, vc), b0, b1, b2, b3);
        mma_bf16(o[2 * jp], pf[kk], b0, b1);
        mma_bf16(o[2 * jp + 1], pf[kk], b2, b3);
      }
    }
    __syncthreads();   // the stage is refilled in the next iteration
  }

  // ---- normalise and store -------------------------------------------------------------------
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
  const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    const int col = 8 * j + 2 * (lane & 3);
    if (r0 < rows_here)
      *reinterpret_cast<uint32_t*>(out + ((size_t)(tok0 + i0 + r0) * H + hq) * D + col) =
          pack_bf16(o[j][0] * inv0, o[j][1] * inv0);
    if (r1 < rows_here)
      *reinterpret_cast<uint32_t*>(out + ((size_t)(tok0 + i0 + r1) * H + hq) * D + col) =
          pack_bf16(o[j][2] * inv1, o[j][3] * inv1);
  }
}

template <int D>
static int launch_prefill(const void* q, void* out, const void* k_cache, const void* v_cache, const int* block_table,
                          int table_width, const int* seq_start, const int* seq_past, int B, int max_new, int H,
                          int G, int window, float scale, cudaStream_t stream) {
  const size_t smem = (size_t)PF_BQ * D * 2 + 4 * (size_t)PF_BK * D * 2;
  auto kernel = attention_prefill_kernel<D>;
  static bool attr_set = false;
  if (!attr_set && smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid(H, (max_new + PF_BQ - 1) / PF_BQ, B);
  launch_pdl(kernel, grid, dim3(PF_THREADS), smem, stream, (const bf16*)q, (bf16*)out, (const bf16*)k_cache, (const bf16*)v_cache,
                                             block_table, table_width, seq_start, seq_past, H, G, window,
                                             scale * 1.4426950408889634f);
  return LLMX_LAUNCH_STATUS();
}

// q, out: bf16 [T, H*D], tokens packed sequence after sequence; seq_start [B+1] offsets into the packed
// tokens; seq_past[b] = position of sequence b's first new token; max_new = most new tokens of a sequence.
// Head sizes 64 and 128; other sizes are refused (the general kernel takes them).
LLMX_API int llmx_attention_prefill(const void* q, void* out, const void* k_cache, const void* v_cache,
                                    const int* block_table, int table_width, const int* seq_start,
                                    const int* seq_past, int B, int max_new, int H, int G, int D, int window,
                                    float scale, cudaStream_t stream) {
  if (B <= 0 || max_new <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || window < 0 || B > 65535 ||
      (max_new + PF_BQ - 1) / PF_BQ > 65535)
    return LLMX_REFUSED(1);
  if (D == 128)
    return launch_prefill<128>(q, out, k_cache, v_cache, block_table, table_width, seq_start, seq_past, B, max_new,
                               H, G, window, scale, stream);
  if (D == 64)
    return launch_prefill<64>(q, out, k_cache, v_cache, block_table, table_width, seq_start, seq_past, B, max_new, H,
                              G, window, scale, stream);
  return LLMX_REFUSED(1);
}
