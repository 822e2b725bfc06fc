// Memory-bound kernels around the matrix products: embedding gather,
// residual add fused with RMSNorm, per-head q/k RMSNorm fused with the NeoX
// rotation and the cache write, and the gated activation.  Sums of squares,
// the residual sum and the rotation are float32 whatever the storage type.
//
// Semantics restated from the reference's scalar ops: rms_norm_mul
// (crates/model/src/ops.rs:40-59), rope_neox (ops.rs:142-159), silu
// (ops.rs:176-178), and the order norm -> rotation -> cache write of
// crates/model/src/qwen35/cpu.rs:295-323.
#include "common.cuh"

__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}


// ---------------------------------------------------------------------------
// Embedding gather: h[t,:] = E[tok_t,:] widened to float32, times `scale` (1 for the dense Qwen3 decoder,
// which has none; a product with 1 is exact).
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ h, int d, int vocab, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);  // never read outside the table
  const TW* row = table + (size_t)tok * d;
  float* out = h + (size_t)t * d;
  if ((d & 3) == 0) {
    // four elements per load, four loads in flight per thread: the row is cold in DRAM
#pragma unroll 4
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
      float4 v = load4(row + i);
      store4(out + i, make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale));
    }
    return;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = to_f32(row[i]) * scale;
}

LLMX_API int llmx_embed(const void* table, int table_dtype, const int* tokens, float* h,
                        int n_tokens, int d, int vocab, float scale, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || vocab <= 0) return LLMX_REFUSED(1);
  const int threads = d >= 1024 ? 256 : 128;
  if (table_dtype == LLMX_F32)
    launch_pdl(embed_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, (const float*)table, tokens, h, d, vocab, scale);
  else if (table_dtype == LLMX_BF16)
    launch_pdl(embed_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, (const bf16*)table, tokens, h, d, vocab, scale);
  else
    return LLMX_REFUSED(2);
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Residual add + RMSNorm.  For output row r (source row t = rows ? rows[r] : r):
//   v = h[t,:] + sum_s delta[s][t,:]      (partials added in the order s = 0..S-1)
//   if write_h: h[t,:] = v
//   out[r,:] = v * (1/sqrt(mean(v^2)+eps)) * gain
// One block per row; a row wider than one pass is staged in shared memory as float32.
// ---------------------------------------------------------------------------
// The thread count and each thread's elements are fixed by d alone, so the reduction order does not depend on the
// batch.  A CTA has at most 512 threads of at most 64 registers: it fits an SM beside the CTAs of the matrix
// product before it, so it is resident, with its weights fetched, when that kernel ends.  Rows up to 8192 wide
// stay in registers from the sum to the store (up to 4 vectors of 4 elements per thread, vector c of thread j at
// column 4 (c nthreads + j)); wider rows are staged in shared memory.

// v += sum_s p[s * stride .. +4), the partials added in the order s = 0..S-1, their loads issued eight at a time
// (a loop of load-then-add would pay one memory round trip per partial).
template <int J = 8, typename TD>
__device__ __forceinline__ void add_partials4(float4& v, const TD* p, int n_split, size_t split_stride) {
  for (int s0 = 0; s0 < n_split; s0 += J) {
    float4 y[J];
#pragma unroll
    for (int j = 0; j < J; ++j)
      if (s0 + j < n_split) y[j] = load4(p + (size_t)(s0 + j) * split_stride);
#pragma unroll
    for (int j = 0; j < J; ++j)
      if (s0 + j < n_split) {
        v.x += y[j].x; v.y += y[j].y; v.z += y[j].z; v.w += y[j].w;
      }
  }
}

// CH > 0: the row fits CH vectors per thread.  CH == 0: any width, staged in shared memory.
// DEEP: many partials and few rows (a decode step): a dozen loads in flight per thread.  Otherwise (one delta,
// thousands of rows) few registers, so that several CTAs share an SM.
template <typename TD, typename TO, int CH, bool DEEP>
__global__ void __launch_bounds__(512)
add_rms_norm_kernel(float* __restrict__ h, const TD* __restrict__ delta, int n_split, size_t split_stride,
                    const int* __restrict__ rows, const float* __restrict__ gain, float eps, TO* __restrict__ out,
                    int d, int write_h) {
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  pdl_launch_dependents();
  // The row index (a step input) and the gain (a weight) do not come from the kernel before: they are
  // fetched while that kernel still runs.
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float* hrow = h + (size_t)t * d;
  const int nthreads = blockDim.x;
  float ss = 0.f;
  if (CH > 0) {
    constexpr int NC = CH > 0 ? CH : 1;
    float4 g[NC], v[NC];
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int i = (c * nthreads + threadIdx.x) * 4;
      g[c] = (out && i < d) ? load4(gain + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int i = (c * nthreads + threadIdx.x) * 4;
      v[c] = i < d ? load4(hrow + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (delta) {
      // partials of every vector of the thread, about a dozen loads in flight (with the row's own above)
      constexpr int J = !DEEP ? 1 : (NC == 1 ? 8 : (NC == 2 ? 5 : 2));
      for (int s0 = 0; s0 < n_split; s0 += J) {
        float4 y[NC][J];
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int i = (c * nthreads + threadIdx.x) * 4;
#pragma unroll
          for (int j = 0; j < J; ++j)
            if (i < d && s0 + j < n_split) y[c][j] = load4(delta + (size_t)(s0 + j) * split_stride + (size_t)t * d + i);
        }
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int i = (c * nthreads + threadIdx.x) * 4;
#pragma unroll
          for (int j = 0; j < J; ++j)
            if (i < d && s0 + j < n_split) {
              v[c].x += y[c][j].x; v[c].y += y[c][j].y; v[c].z += y[c][j].z; v[c].w += y[c][j].w;
            }
        }
      }
      if (write_h) {
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          const int i = (c * nthreads + threadIdx.x) * 4;
          if (i < d) store4(hrow + i, v[c]);
        }
      }
    }
#pragma unroll
    for (int c = 0; c < NC; ++c) {        // dead vectors are zero
      ss += v[c].x * v[c].x;
      ss += v[c].y * v[c].y;
      ss += v[c].z * v[c].z;
      ss += v[c].w * v[c].w;
    }
    const float total = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(total / (float)d + eps);
    if (out) {
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int i = (c * nthreads + threadIdx.x) * 4;
        if (i < d)
          store4(out + (size_t)r * d + i, make_float4((v[c].x * scale) * g[c].x, (v[c].y * scale) * g[c].y,
                                                      (v[c].z * scale) * g[c].z, (v[c].w * scale) * g[c].w));
      }
    }
    return;
  }
  pdl_wait();
  if ((d & 3) == 0) {
    for (int i = threadIdx.x * 4; i < d; i += nthreads * 4) {
      float4 v = load4(hrow + i);
      if (delta) {
        add_partials4<DEEP ? 8 : 1>(v, delta + (size_t)t * d + i, n_split, split_stride);
        if (write_h) store4(hrow + i, v);
      }
      store4(row_buf + i, v);
      ss += v.x * v.x;
      ss += v.y * v.y;
      ss += v.z * v.z;
      ss += v.w * v.w;
    }
  } else {
    for (int i = threadIdx.x; i < d; i += nthreads) {
      float v = hrow[i];
      if (delta) {
        const TD* p = delta + (size_t)t * d + i;
        for (int s = 0; s < n_split; ++s) v += to_f32(p[s * split_stride]);
        if (write_h) hrow[i] = v;
      }
      row_buf[i] = v;
      ss += v * v;
    }
  }
  const float total = block_sum(ss, red);
  const float scale = 1.0f / sqrtf(total / (float)d + eps);
  if (out) {
    TO* orow = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += nthreads) orow[i] = from_f32<TO>((row_buf[i] * scale) * gain[i]);
  }
}

// (vectors per thread, threads) for a row of d elements; 0 vectors: the staged path
static void norm_shape(int d, int& ch, int& threads) {
  const int vecs = (d + 3) / 4;
  ch = 0;
  threads = 512;
  if ((d & 3) == 0 && vecs <= 4 * 512) {
    ch = vecs <= 512 ? 1 : (vecs <= 1024 ? 2 : 4);
    threads = ((vecs + ch - 1) / ch + 31) / 32 * 32;
    if (threads < 64) threads = 64;
  }
}

template <typename TD, typename TO>
static int launch_add_rms_norm(float* h, const void* delta, int n_split, size_t split_stride, const int* rows,
                               int n_rows, const float* gain, float eps, void* out, int d, int write_h,
                               cudaStream_t stream) {
  int ch, threads;
  norm_shape(d, ch, threads);
  const bool deep = delta && n_split > 1;
#define GO(CH, SMEM)                                                                                              \
  do {                                                                                                            \
    if (deep)                                                                                                     \
      launch_pdl(add_rms_norm_kernel<TD, TO, CH, true>, dim3(n_rows), dim3(threads), SMEM, stream, h,            \
                 (const TD*)delta, n_split, split_stride, rows, gain, eps, (TO*)out, d, write_h);                \
    else                                                                                                          \
      launch_pdl(add_rms_norm_kernel<TD, TO, CH, false>, dim3(n_rows), dim3(threads), SMEM, stream, h,           \
                 (const TD*)delta, n_split, split_stride, rows, gain, eps, (TO*)out, d, write_h);                \
  } while (0)
  if (ch == 1) GO(1, 0);
  else if (ch == 2) GO(2, 0);
  else if (ch == 4) GO(4, 0);
  else {
    const size_t smem = (size_t)d * sizeof(float);
    if (smem > 48 * 1024) {
      if (smem > 200 * 1024) return LLMX_REFUSED(3);
      cudaError_t e = cudaFuncSetAttribute(add_rms_norm_kernel<TD, TO, 0, true>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(add_rms_norm_kernel<TD, TO, 0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    GO(0, smem);
  }
#undef GO
  return LLMX_LAUNCH_STATUS();
}

LLMX_API int llmx_add_rms_norm(float* h, const void* delta, int delta_dtype, int n_split, long long split_stride,
                               const int* rows, int n_rows, const float* gain, float eps, void* out,
                               int out_dtype, int d, int write_h, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (d <= 0 || (delta && n_split < 1)) return LLMX_REFUSED(1);
#define CASE(TD, TO) \
  return launch_add_rms_norm<TD, TO>(h, delta, n_split, (size_t)split_stride, rows, n_rows, gain, eps, out, d, write_h, stream)
  if (delta_dtype == LLMX_F32 && out_dtype == LLMX_F32) CASE(float, float);
  if (delta_dtype == LLMX_F32 && out_dtype == LLMX_BF16) CASE(float, bf16);
  if (delta_dtype == LLMX_BF16 && out_dtype == LLMX_F32) CASE(bf16, float);
  if (delta_dtype == LLMX_BF16 && out_dtype == LLMX_BF16) CASE(bf16, bf16);
#undef CASE
  return LLMX_REFUSED(2);
}

// ---------------------------------------------------------------------------
// Residual add and the first half of the RMSNorm, spread over many CTAs, for a step of few tokens.  One CTA
// per (token, slice of ADD_SLICE columns):
//   v = h[t,:] + sum_s delta[s][t,:]  (in the order s = 0..S-1, as add_rms_norm);  h[t,:] = v
//   x[t,:] = bf16(v * gain);  sumsq[slice][t] = sum of v^2 over the slice
// The matrix product that reads x multiplies its output row t by 1/sqrt(sum_slices sumsq / d + eps) (gemm_tc.cu,
// TcScale), which completes the norm.  With one CTA per row (add_rms_norm) a decode step's partial sums are
// loaded by as many SMs as the batch has tokens; here every SM takes part and no CTA waits for another.
// ---------------------------------------------------------------------------
#define ADD_SLICE 512

template <typename TD>
__global__ void __launch_bounds__(ADD_SLICE / 4)
add_gain_sumsq_kernel(float* __restrict__ h, const TD* __restrict__ delta, int n_split, size_t split_stride,
                      const float* __restrict__ gain, bf16* __restrict__ x, float* __restrict__ sumsq,
                      int sumsq_stride, int d) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int t = blockIdx.y, i = (blockIdx.x * (ADD_SLICE / 4) + threadIdx.x) * 4;
  const bool live = i < d;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 g = live ? load4(gain + i) : zero;      // a weight: fetched while the kernel before still runs
  pdl_wait();
  float4 v = zero;
  if (live) {
    float* hp = h + (size_t)t * d + i;
    v = load4(hp);
    if (delta) {
      add_partials4<16>(v, delta + (size_t)t * d + i, n_split, split_stride);
      store4(hp, v);
    }
    store4(x + (size_t)t * d + i, make_float4(v.x * g.x, v.y * g.y, v.z * g.z, v.w * g.w));
  }
  float ss = v.x * v.x;
  ss += v.y * v.y;
  ss += v.z * v.z;
  ss += v.w * v.w;
  const float total = block_sum(ss, red);
  if (threadIdx.x == 0) sumsq[(size_t)blockIdx.x * sumsq_stride + t] = total;
}

// h float32 [T,d] (d a multiple of 4); delta nullptr or [n_split][T,d]; x bf16 [T,d];
// sumsq float32 [ceil(d/ADD_SLICE)][sumsq_stride >= T].
LLMX_API int llmx_add_gain_sumsq(float* h, const void* delta, int delta_dtype, int n_split, long long split_stride,
                                 const float* gain, void* x, float* sumsq, int sumsq_stride, int n_tokens, int d,
                                 cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (d <= 0 || (d & 3) || n_tokens > 65535 || sumsq_stride < n_tokens || (delta && n_split < 1)) return LLMX_REFUSED(1);
  dim3 grid((d + ADD_SLICE - 1) / ADD_SLICE, n_tokens);
  if (delta_dtype == LLMX_F32)
    launch_pdl(add_gain_sumsq_kernel<float>, grid, dim3(ADD_SLICE / 4), 0, stream, h, (const float*)delta, n_split,
               (size_t)split_stride, gain, (bf16*)x, sumsq, sumsq_stride, d);
  else if (delta_dtype == LLMX_BF16)
    launch_pdl(add_gain_sumsq_kernel<bf16>, grid, dim3(ADD_SLICE / 4), 0, stream, h, (const bf16*)delta, n_split,
               (size_t)split_stride, gain, (bf16*)x, sumsq, sumsq_stride, d);
  else
    return LLMX_REFUSED(2);
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Per-head RMSNorm of q and k, NeoX rotation of both, and the cache write of
// k and v.  Input qkv [T, (H+2G)*D]: q heads, then k heads, then v heads.
// One warp per (token, head).  The normalised head is staged in shared memory
// so that a dim can read its rotation partner (i, i + n_rot/2) at any D.
// cos/sin tables are [max_pos, n_rot/2] float32, made on the host in float64.
// ---------------------------------------------------------------------------
#define QKV_WARPS 4

// DEEP: a decode step (few tokens, split partials): one head per warp, the partials' loads batched.  Otherwise
// (a prompt): a warp takes QKV_SPW heads of its token one after another, so that the token's position, block
// table entry, gains and rotation rows are fetched once for all of them, and their loads go out together.
#define QKV_SPW 4

template <typename TIN, typename TA, typename TC, bool DEEP>
__global__ void qk_norm_rope_cache_kernel(const TIN* __restrict__ qkv, int n_split, size_t split_stride,
                                          TA* __restrict__ q_out,
                                          TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                                          const int* __restrict__ block_table, int table_width,
                                          const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                          const float* __restrict__ q_gain, const float* __restrict__ k_gain,
                                          float eps, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, int n_rot, int H, int G, int D,
                                          int write_cache) {
  constexpr int SPW = DEEP ? 1 : QKV_SPW;
  extern __shared__ float head_buf[];
  pdl_launch_dependents();
  // Positions, block table, gains and rotation tables are step inputs or weights, not results of the kernel
  // before: they are fetched ahead of the dependency wait, which only the qkv values need.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;                        // tokens on x: a step may bring more than 65535
  const int slot0 = (blockIdx.y * QKV_WARPS + warp) * SPW;   // the warp's first head of the fused row
  const int n_slots = write_cache ? H + 2 * G : H;
  if (slot0 >= n_slots) return;
  float* buf = head_buf + warp * D;
  const TIN* tok = qkv + (size_t)t * (H + 2 * G) * D;
  const int pos = token_pos[t];
  int page = 0;
  if (slot0 + SPW > H) page = block_table[(size_t)token_seq[t] * table_width + pos / LLMX_PAGE];
  auto cache_row_of = [&](int slot) -> TC* {        // slot >= H: a k head, then the v heads
    const bool is_k = slot < H + G;
    return (is_k ? k_cache : v_cache) + cache_row_offset(page, is_k ? slot - H : slot - H - G, pos % LLMX_PAGE, G, D);
  };

  if (D == 128 && n_rot == 128) {
    // Head size 128 with full rotation: a lane owns dims 4*lane..4*lane+3, read and written as one
    // vector; the rotation partner (dim +-64) lives in lane +-16 and comes by shuffle.
    const int d0 = 4 * lane;
    const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 gq = q_gain ? load4(q_gain + d0) : one, gk = k_gain ? load4(k_gain + d0) : one;
    const float4 cs = load4(cos_t + (size_t)pos * 64 + (d0 & 63)), sn = load4(sin_t + (size_t)pos * 64 + (d0 & 63));
    pdl_wait();
    float4 xs[SPW];
#pragma unroll
    for (int j = 0; j < SPW; ++j) {
      if (slot0 + j < n_slots) {
        const TIN* src = tok + (size_t)(slot0 + j) * D;
        xs[j] = load4(src + d0);
        add_partials4<DEEP ? 8 : 1>(xs[j], src + split_stride + d0, n_split - 1, split_stride);
      }
    }
#pragma unroll
    for (int j = 0; j < SPW; ++j) {
      const int slot = slot0 + j;
      if (slot >= n_slots) break;
      float4 x = xs[j];
      const bool is_q = slot < H, is_k = !is_q && slot < H + G;
      if (!is_q && !is_k) {  // v: stored as it is
        store4(cache_row_of(slot) + d0, x);
        continue;
      }
      if (is_q ? q_gain != nullptr : k_gain != nullptr) {
        const float4 gn = is_q ? gq : gk;
        const float ssq = warp_sum(x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w);
        const float scale = 1.0f / sqrtf(ssq / 128.0f + eps);
        x.x = (x.x * scale) * gn.x; x.y = (x.y * scale) * gn.y; x.z = (x.z * scale) * gn.z; x.w = (x.w * scale) * gn.w;
      }
      float4 p;
      p.x = __shfl_xor_sync(0xffffffffu, x.x, 16);
      p.y = __shfl_xor_sync(0xffffffffu, x.y, 16);
      p.z = __shfl_xor_sync(0xffffffffu, x.z, 16);
      p.w = __shfl_xor_sync(0xffffffffu, x.w, 16);
      float4 r;
      if (lane < 16) {   // dims i < 64: x_i cos - x_{i+64} sin
        r = make_float4(x.x * cs.x - p.x * sn.x, x.y * cs.y - p.y * sn.y, x.z * cs.z - p.z * sn.z, x.w * cs.w - p.w * sn.w);
      } else {           // dims i + 64: x_i sin + x_{i+64} cos
        r = make_float4(p.x * sn.x + x.x * cs.x, p.y * sn.y + x.y * cs.y, p.z * sn.z + x.z * cs.z, p.w * sn.w + x.w * cs.w);
      }
      if (is_q) store4(q_out + (size_t)t * H * D + (size_t)slot * D + d0, r);
      else store4(cache_row_of(slot) + d0, r);
    }
    return;
  }

  pdl_wait();
  for (int j = 0; j < SPW; ++j) {
    const int slot = slot0 + j;
    if (slot >= n_slots) break;
    const TIN* src = tok + (size_t)slot * D;
    // the head's values: one tensor, or split partials added in order
    auto value = [&](int i) {
      float v = to_f32(src[i]);
      for (int s = 1; s < n_split; ++s) v += to_f32(src[s * split_stride + i]);
      return v;
    };
    const bool is_q = slot < H, is_k = !is_q && slot < H + G;
    TC* cache_row = is_q ? nullptr : cache_row_of(slot);
    if (!is_q && !is_k) {  // v: stored as it is
      for (int i = lane; i < D; i += 32) cache_row[i] = from_f32<TC>(value(i));
      continue;
    }
    const float* gain = is_q ? q_gain : k_gain;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float v = value(i);
      buf[i] = v;
      ss += v * v;
    }
    if (gain) {
      const float scale = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
      for (int i = lane; i < D; i += 32) buf[i] = (buf[i] * scale) * gain[i];
    }
    __syncwarp();
    const int half = n_rot >> 1;
    const float* c = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* sv = sin_t ? sin_t + (size_t)pos * half : nullptr;
    TA* qrow = is_q ? q_out + (size_t)t * H * D + (size_t)slot * D : nullptr;
    for (int i = lane; i < D; i += 32) {
      float v = buf[i];
      if (i < half) {
        v = buf[i] * c[i] - buf[i + half] * sv[i];
      } else if (i < n_rot) {
        v = buf[i - half] * sv[i - half] + buf[i] * c[i - half];
      }
      if (is_q) qrow[i] = from_f32<TA>(v);
      else cache_row[i] = from_f32<TC>(v);
    }
    __syncwarp();   // buf is filled again for the warp's next head
  }
}

// The same for prompts when everything is bfloat16, the head size is 128 and the rotation is full: half a
// warp per head, a lane owns eight consecutive dims (one 16-byte load, one 16-byte store); the rotation
// partner (dim +-64) lives eight lanes away.  A warp takes eight heads of its token, two at a time.
#define QKV8_PER_WARP 8

__global__ void qk_norm_rope_cache_bf16_d128_kernel(const bf16* __restrict__ qkv, bf16* __restrict__ q_out,
                                                    bf16* __restrict__ k_cache, bf16* __restrict__ v_cache,
                                                    const int* __restrict__ block_table, int table_width,
                                                    const int* __restrict__ token_seq,
                                                    const int* __restrict__ token_pos,
                                                    const float* __restrict__ q_gain,
                                                    const float* __restrict__ k_gain, float eps,
                                                    const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                    int H, int G, int write_cache) {
  constexpr int D = 128;
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int half = lane >> 4, l16 = lane & 15, d0 = 8 * l16;
  const unsigned mask = half ? 0xffff0000u : 0x0000ffffu;      // the lanes that share this lane's head
  const int t = blockIdx.x;
  const int slot_base = (blockIdx.y * QKV_WARPS + warp) * QKV8_PER_WARP;
  const int n_slots = write_cache ? H + 2 * G : H;
  if (slot_base >= n_slots) return;
  // step inputs and weights first: they do not wait for the kernel before
  const int pos = token_pos[t];
  int page = 0;
  if (slot_base + QKV8_PER_WARP > H) page = block_table[(size_t)token_seq[t] * table_width + pos / LLMX_PAGE];
  float gq[8], gk[8], cs[8], sn[8];
  {
    const float4 one = make_float4(1.f, 1.f, 1.f, 1.f);
    const float4 a0 = q_gain ? load4(q_gain + d0) : one, a1 = q_gain ? load4(q_gain + d0 + 4) : one;
    const float4 b0 = k_gain ? load4(k_gain + d0) : one, b1 = k_gain ? load4(k_gain + d0 + 4) : one;
    const float4 c0 = load4(cos_t + (size_t)pos * 64 + (d0 & 63)), c1 = load4(cos_t + (size_t)pos * 64 + (d0 & 63) + 4);
    const float4 s0 = load4(sin_t + (size_t)pos * 64 + (d0 & 63)), s1 = load4(sin_t + (size_t)pos * 64 + (d0 & 63) + 4);
    gq[0] = a0.x; gq[1] = a0.y; gq[2] = a0.z; gq[3] = a0.w; gq[4] = a1.x; gq[5] = a1.y; gq[6] = a1.z; gq[7] = a1.w;
    gk[0] = b0.x; gk[1] = b0.y; gk[2] = b0.z; gk[3] = b0.w; gk[4] = b1.x; gk[5] = b1.y; gk[6] = b1.z; gk[7] = b1.w;
    cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
    sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
  }
  pdl_wait();
  const bf16* tok = qkv + (size_t)t * (H + 2 * G) * D;
  uint4 raw[QKV8_PER_WARP / 2];
#pragma unroll
  for (int j = 0; j < QKV8_PER_WARP / 2; ++j) {
    const int slot = slot_base + 2 * j + half;
    if (slot < n_slots) raw[j] = *reinterpret_cast<const uint4*>(tok + (size_t)slot * D + d0);
  }
#pragma unroll
  for (int j = 0; j < QKV8_PER_WARP / 2; ++j) {
    const int slot = slot_base + 2 * j + half;                 // the same for the sixteen lanes of a half
    if (slot >= n_slots) continue;
    const bool is_q = slot < H, is_k = !is_q && slot < H + G;
    bf16* dst;
    if (is_q) {
      dst = q_out + (size_t)t * H * D + (size_t)slot * D + d0;
    } else {
      const int g = is_k ? slot - H : slot - H - G;
      dst = (is_k ? k_cache : v_cache) + cache_row_offset(page, g, pos % LLMX_PAGE, G, D) + d0;
    }
    if (!is_q && !is_k) {                                      // v: stored as it is
      *reinterpret_cast<uint4*>(dst) = raw[j];
      continue;
    }
    float x[8];
    {
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h2[i]);
        x[2 * i] = f.x;
        x[2 * i + 1] = f.y;
      }
    }
    const float* gain = is_q ? gq : gk;
    if (is_q ? q_gain != nullptr : k_gain != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
#pragma unroll
      for (int sh = 8; sh > 0; sh >>= 1) ss += __shfl_xor_sync(mask, ss, sh);
      const float scale = 1.0f / sqrtf(ss / 128.0f + eps);
#pragma unroll
      for (int i = 0; i < 8; ++i) x[i] = (x[i] * scale) * gain[i];
    }
    uint32_t packed[4];
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const float p0 = __shfl_xor_sync(mask, x[i], 8), p1 = __shfl_xor_sync(mask, x[i + 1], 8);
      float r0, r1;
      if (l16 < 8) {   // dims i < 64: x_i cos - x_{i+64} sin
        r0 = x[i] * cs[i] - p0 * sn[i];
        r1 = x[i + 1] * cs[i + 1] - p1 * sn[i + 1];
      } else {         // dims i + 64: x_i sin + x_{i+64} cos
        r0 = p0 * sn[i] + x[i] * cs[i];
        r1 = p1 * sn[i + 1] + x[i + 1] * cs[i + 1];
      }
      __nv_bfloat162 h = __floats2bfloat162_rn(r0, r1);
      packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
}

LLMX_API int llmx_qk_norm_rope_cache(const void* qkv, int in_dtype, int n_split, long long split_stride, void* q_out,
                                     int act_dtype, void* k_cache, void* v_cache, int cache_dtype,
                                     const int* block_table, int table_width, const int* token_seq,
                                     const int* token_pos, const float* q_gain, const float* k_gain, float eps,
                                     const float* cos_t, const float* sin_t, int n_rot, int n_tokens, int H, int G,
                                     int D, int write_cache, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || D <= 0 || n_rot < 0 || n_rot > D || (n_rot & 1) || n_split < 1) return LLMX_REFUSED(1);
  if (n_rot > 0 && (!cos_t || !sin_t)) return LLMX_REFUSED(4);
  const int n_slots = write_cache ? H + 2 * G : H;
  if (n_split == 1 && in_dtype == LLMX_BF16 && act_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16 && D == 128 &&
      n_rot == 128 && n_tokens > 64 && !(((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_cache | (uintptr_t)v_cache) & 15)) {
    const int per_cta = QKV_WARPS * QKV8_PER_WARP;
    launch_pdl(qk_norm_rope_cache_bf16_d128_kernel, dim3(n_tokens, (n_slots + per_cta - 1) / per_cta),
               dim3(QKV_WARPS * 32), 0, stream, (const bf16*)qkv, (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache,
               block_table, table_width, token_seq, token_pos, q_gain, k_gain, eps, cos_t, sin_t, H, G, write_cache);
    return LLMX_LAUNCH_STATUS();
  }
  const bool deep = n_split > 2;
  const int per_cta = QKV_WARPS * (deep ? 1 : QKV_SPW);
  dim3 grid(n_tokens, (n_slots + per_cta - 1) / per_cta);
  const size_t smem = (size_t)QKV_WARPS * D * sizeof(float);
  if (smem > 48 * 1024) return LLMX_REFUSED(3);
  // many partials (a decode step): their loads batched; one tensor (a prompt): few registers, many warps per SM
#define CASE(TIN, TA, TC)                                                                                          \
  do {                                                                                                             \
    if (deep)                                                                                                      \
      launch_pdl(qk_norm_rope_cache_kernel<TIN, TA, TC, true>, grid, dim3(QKV_WARPS * 32), smem, stream,           \
        (const TIN*)qkv, n_split, (size_t)split_stride, (TA*)q_out, (TC*)k_cache, (TC*)v_cache, block_table,        \
        table_width, token_seq, token_pos, q_gain, k_gain, eps, cos_t, sin_t, n_rot, H, G, D, write_cache);         \
    else                                                                                                           \
      launch_pdl(qk_norm_rope_cache_kernel<TIN, TA, TC, false>, grid, dim3(QKV_WARPS * 32), smem, stream,          \
        (const TIN*)qkv, n_split, (size_t)split_stride, (TA*)q_out, (TC*)k_cache, (TC*)v_cache, block_table,        \
        table_width, token_seq, token_pos, q_gain, k_gain, eps, cos_t, sin_t, n_rot, H, G, D, write_cache);         \
  } while (0)
  const int key = in_dtype * 4 + act_dtype * 2 + cache_dtype;
  switch (key) {
    case 0: CASE(float, float, float); break;
    case 1: CASE(float, float, bf16); break;
    case 2: CASE(float, bf16, float); break;
    case 3: CASE(float, bf16, bf16); break;
    case 6: CASE(bf16, bf16, float); break;
    case 7: CASE(bf16, bf16, bf16); break;
    default: return LLMX_REFUSED(2);
  }
#undef CASE
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Gated activation: act[t,f] = silu(g) * u with g = sum_s gu[s][t,f] and
// u = sum_s gu[s][t,F+f]; silu(x) = x / (1 + exp(-x)) in float32.
// ---------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void silu_gate_kernel(const TI* __restrict__ gu, int n_split, size_t split_stride,
                                 TO* __restrict__ act, int n_tokens, int F, int block) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t n = (size_t)n_tokens * F;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < n; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / F, f = idx - t * F;
    // block == 0: columns [gate 0..F) [up 0..F).  block > 0: blocks of `block` gate columns followed by the
    // `block` up columns of the same features.
    const size_t gcol = block > 0 ? (f / block) * 2 * block + f % block : f;
    const size_t ucol = block > 0 ? gcol + block : f + F;
    const TI* p = gu + t * 2 * (size_t)F;
    float g = 0.f, u = 0.f;
    for (int s = 0; s < n_split; ++s) {
      g += to_f32(p[s * split_stride + gcol]);
      u += to_f32(p[s * split_stride + ucol]);
    }
    act[idx] = from_f32<TO>((g / (1.0f + expf(-g))) * u);
  }
}

LLMX_API int llmx_silu_gate(const void* gu, int in_dtype, int n_split, long long split_stride, void* act,
                            int out_dtype, int n_tokens, int F, int block, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (F <= 0 || n_split < 1 || block < 0 || (block > 0 && F % block)) return LLMX_REFUSED(1);
  const size_t n = (size_t)n_tokens * F;
  const int threads = 256;
  const int blocks = (int)((n + threads - 1) / threads < 148 * 16 ? (n + threads - 1) / threads : 148 * 16);
#define CASE(TI, TO)                                                                                        \
  launch_pdl(silu_gate_kernel<TI, TO>, dim3(blocks), dim3(threads), 0, stream, (const TI*)gu, n_split,      \
             (size_t)split_stride, (TO*)act, n_tokens, F, block)
  if (in_dtype == LLMX_F32 && out_dtype == LLMX_F32) CASE(float, float);
  else if (in_dtype == LLMX_F32 && out_dtype == LLMX_BF16) CASE(float, bf16);
  else if (in_dtype == LLMX_BF16 && out_dtype == LLMX_BF16) CASE(bf16, bf16);
  else if (in_dtype == LLMX_BF16 && out_dtype == LLMX_F32) CASE(bf16, float);
  else return LLMX_REFUSED(2);
#undef CASE
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Sum of split partials into one tensor: out[i] = sum_s in[s][i].
// ---------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void sum_splits_kernel(const TI* __restrict__ in, int n_split, size_t split_stride, TO* __restrict__ out,
                                  size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < n_split; ++s) v += to_f32(in[s * split_stride + i]);
    out[i] = from_f32<TO>(v);
  }
}

LLMX_API int llmx_sum_splits(const void* in, int in_dtype, int n_split, long long split_stride, void* out,
                             int out_dtype, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n_split < 1) return LLMX_REFUSED(1);
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
#define CASE(TI, TO) \
  launch_pdl(sum_splits_kernel<TI, TO>, dim3(blocks), dim3(threads), 0, stream, (const TI*)in, n_split, (size_t)split_stride, (TO*)out, (size_t)n)
  if (in_dtype == LLMX_F32 && out_dtype == LLMX_F32) CASE(float, float);
  else if (in_dtype == LLMX_F32 && out_dtype == LLMX_BF16) CASE(float, bf16);
  else if (in_dtype == LLMX_BF16 && out_dtype == LLMX_BF16) CASE(bf16, bf16);
  else if (in_dtype == LLMX_BF16 && out_dtype == LLMX_F32) CASE(bf16, float);
  else return LLMX_REFUSED(2);
#undef CASE
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Soft cap of logits, in place: x = cap * tanh(x / cap), float32.
// ---------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, size_t n, float cap) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}

LLMX_API int llmx_softcap(float* x, long long n, float cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!(cap > 0.f)) return LLMX_REFUSED(1);
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  launch_pdl(softcap_kernel, dim3(blocks), dim3(threads), 0, stream, x, (size_t)n, cap);
  return LLMX_LAUNCH_STATUS();
}
