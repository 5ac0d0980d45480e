// Pointwise producers of the repaired linears' inputs: each writes its bf16 result once and, in the same
// pass, reduces max|y| so that the following NVFP4 quantizer starts from a known tensor factor instead of
// re-reading its input.
//
//   tw_activate       relu(a)^2, a*b (thunderworld_fp4/_fusion.py:15-34 pointwise_amax / activate_with_factor:
//                     fp32 math, one bf16 rounding, factor = max|y| / 2688 or 1 for an all-zero tensor as in
//                     finish_amax, _linear_kernels.py:17-19), and tanh-GELU for the DiT step
//   tw_rms_norm       RMSNorm with optional weight (cosmos/norm_fusion.py:23-43) and optional AdaLN
//                     modulation y = norm * (1 + scale[b]) + shift[b]
//   tw_rms_norm_heads RMSNorm over head_dim = 128 rows of a strided [tokens, heads, 128] view (q / k norm)
//   tw_rope_heads     exact-rounding rotary embedding of such rows (cosmos/pipeline_tuning.py:42-63), optionally
//                     after the head norm in the same pass
//   tw_gate_residual  x += gate[b] * y
//
// All are HBM-bound: 16-byte loads and stores, every input element read once. The factor is finished by the
// last CTA to retire (ticket counter in an 8-byte scratch that the kernel leaves zeroed), so no second launch
// and no memset are needed and the sequence can be captured in a CUDA Graph.
#include "tw_common.cuh"
#include "../../include/twb200.h"

namespace {

constexpr float FACTOR_DIVISOR = 2688.f;       // 6 * 448: largest E2M1 value times largest E4M3 scale

__device__ __forceinline__ void unpack8(const uint4& v, float (&x)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = tw::bf16_bits_to_float(w[i] & 0xffffu);
    x[2 * i + 1] = tw::bf16_bits_to_float(w[i] >> 16);
  }
}
// Rounds to bf16, packs, and folds |rounded value| into `peak`.
__device__ __forceinline__ uint4 pack8(const float (&y)[8], float& peak) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(y[2 * i], y[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&b);
    peak = fmaxf(peak, fmaxf(fabsf(__low2float(b)), fabsf(__high2float(b))));
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block maximum -> global maximum (bit pattern of a non-negative float orders like the float); the last
// CTA to take a ticket writes stats = {factor, max|y|} and clears the scratch for the next call.
__device__ __forceinline__ void finish_factor(float peak, unsigned* scratch, float* stats) {
  __shared__ float part[32];
  __shared__ bool last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = (blockDim.x + 31) >> 5;
  peak = warp_max(peak);
  if (lane == 0) part[warp] = peak;
  __syncthreads();
  if (warp == 0) {
    peak = warp_max(lane < warps ? part[lane] : 0.f);
    if (lane == 0) {
      atomicMax(scratch, __float_as_uint(peak));
      __threadfence();
      last = atomicAdd(scratch + 1, 1u) == gridDim.x * gridDim.y - 1;
      if (last) {
        __threadfence();
        const float top = __uint_as_float(atomicExch(scratch, 0u));
        stats[0] = top > 0.f ? __fdiv_rn(top, FACTOR_DIVISOR) : 1.f;
        stats[1] = top;
        scratch[1] = 0u;
      }
    }
  }
}

using tw::gelu_tanh;

// ---- activation -----------------------------------------------------------------------------
template <int MODE>
__global__ void __launch_bounds__(256) activate_kernel(const uint4* __restrict__ a, const uint4* __restrict__ b,
                                                       uint4* __restrict__ y, long long vecs, unsigned* scratch, float* stats) {
  float peak = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.x * blockDim.x) {
    float x[8], r[8];
    unpack8(__ldg(a + i), x);
    if (MODE == TW_ACT_RELU2) {
#pragma unroll
      for (int j = 0; j < 8; ++j) { const float t = fmaxf(x[j], 0.f); r[j] = __fmul_rn(t, t); }
    } else if (MODE == TW_ACT_MUL) {
      float z[8];
      unpack8(__ldg(b + i), z);
#pragma unroll
      for (int j = 0; j < 8; ++j) r[j] = __fmul_rn(x[j], z[j]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) r[j] = gelu_tanh(x[j]);
    }
    y[i] = pack8(r, peak);
  }
  if (stats) finish_factor(peak, scratch, stats);
}

// ---- RMSNorm over a full hidden row (one CTA per row, the row stays in registers) -----------------
template <int VPT>   // 16-byte vectors per thread, 256 threads
__global__ void __launch_bounds__(256) rms_norm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ weight,
                                                       const uint4* __restrict__ shift, const uint4* __restrict__ scale,
                                                       uint4* __restrict__ y, int hidden_vecs, int rows_per_batch, float eps,
                                                       unsigned* scratch, float* stats) {
  __shared__ float part[8];
  const int row = blockIdx.x;
  const uint4* src = x + (size_t)row * hidden_vecs;
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c = threadIdx.x + j * 256;
    if (c < hidden_vecs) {
      unpack8(__ldg(src + c), v[j]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = __fmaf_rn(v[j][i], v[j][i], ss);
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  ss = part[0] + part[1] + part[2] + part[3] + part[4] + part[5] + part[6] + part[7];
  const float rstd = rsqrtf(ss / (float)(hidden_vecs * 8) + eps);
  const size_t mod = (size_t)(row / rows_per_batch) * hidden_vecs;
  float peak = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int c = threadIdx.x + j * 256;
    if (c < hidden_vecs) {
      float r[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) r[i] = v[j][i] * rstd;
      if (weight) {
        float w[8];
        unpack8(__ldg(weight + c), w);
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] *= w[i];
      }
      if (scale) {
        float sc[8], sh[8];
        unpack8(__ldg(scale + mod + c), sc);
        unpack8(__ldg(shift + mod + c), sh);
#pragma unroll
        for (int i = 0; i < 8; ++i) r[i] = __fmaf_rn(r[i], 1.f + sc[i], sh[i]);
      }
      y[(size_t)row * hidden_vecs + c] = pack8(r, peak);
    }
  }
  if (stats) {
    __syncthreads();            // `part` is reused by nothing below, but keep the phases apart
    finish_factor(peak, scratch, stats);
  }
}

// ---- RMSNorm and / or rotary embedding over 128-wide head rows of a strided view: 8 lanes per row, 32 rows per CTA
// RoPE follows the reference's exact-rounding kernel (thunderworld_fp4/cosmos/pipeline_tuning.py:42-55):
// y[d] = bf16( bf16(x[d] c[d]) + bf16(rot[d] s[d]) ), rot[d] = -x[d + 64] for d < 64, x[d - 64] otherwise, with
// x the bf16 output of the norm when both run here (the same roundings as two separate kernels, one pass less).
// A lane holds 16 consecutive channels, so its rotation partners sit in lane ^ 4 at the same positions.
template <bool NORM, bool ROPE, typename TableT>
__global__ void __launch_bounds__(256) head_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                        long long rows, int heads, long long stride_token,
                                                        long long stride_head, float eps, const TableT* __restrict__ cos_t,
                                                        const TableT* __restrict__ sin_t, long long table_rows) {
  const long long row = (long long)blockIdx.x * 32 + (threadIdx.x >> 3);      // row = token * heads + head
  const int lane8 = threadIdx.x & 7;
  float v[16];
  const bool live = row < rows;
  const long long token = live ? row / heads : 0, head = live ? row % heads : 0;
  if (live) {
    const uint4* src = reinterpret_cast<const uint4*>(x + token * stride_token + head * stride_head + lane8 * 16);
    float lo[8], hi[8];
    unpack8(__ldg(src), lo);
    unpack8(__ldg(src + 1), hi);
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[i] = lo[i]; v[8 + i] = hi[i]; }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = 0.f;
  }
  if (NORM) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) ss = __fmaf_rn(v[i], v[i], ss);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss * (1.f / 128.f) + eps);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = ROPE ? __bfloat162float(__float2bfloat16_rn(v[i] * rstd)) : v[i] * rstd;
  }
  if (ROPE) {
    // the 16 table entries of this lane, fetched as 16-byte vectors (the tables are rows of 128 entries, so a
    // lane's slice is 16-byte aligned for both table types)
    const long long t = (token % table_rows) * 128 + lane8 * 16;
    float c[16], sn[16];
    if (live) {
      if (sizeof(TableT) == 4) {
        const float4* c4 = reinterpret_cast<const float4*>(cos_t + t);
        const float4* s4 = reinterpret_cast<const float4*>(sin_t + t);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 a = __ldg(c4 + i), b = __ldg(s4 + i);
          c[4 * i] = a.x; c[4 * i + 1] = a.y; c[4 * i + 2] = a.z; c[4 * i + 3] = a.w;
          sn[4 * i] = b.x; sn[4 * i + 1] = b.y; sn[4 * i + 2] = b.z; sn[4 * i + 3] = b.w;
        }
      } else {
        const uint4* c4 = reinterpret_cast<const uint4*>(cos_t + t);
        const uint4* s4 = reinterpret_cast<const uint4*>(sin_t + t);
        unpack8(__ldg(c4), *reinterpret_cast<float(*)[8]>(&c[0]));
        unpack8(__ldg(c4 + 1), *reinterpret_cast<float(*)[8]>(&c[8]));
        unpack8(__ldg(s4), *reinterpret_cast<float(*)[8]>(&sn[0]));
        unpack8(__ldg(s4 + 1), *reinterpret_cast<float(*)[8]>(&sn[8]));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) { c[i] = 0.f; sn[i] = 0.f; }
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float partner = __shfl_xor_sync(0xffffffffu, v[i], 4);
      const float rot = lane8 < 4 ? -partner : partner;
      const float pc = __bfloat162float(__float2bfloat16_rn(__fmul_rn(v[i], c[i])));
      const float qs = __bfloat162float(__float2bfloat16_rn(__fmul_rn(rot, sn[i])));
      v[i] = __fadd_rn(pc, qs);
    }
  }
  if (live) {
    float lo[8], hi[8], unused = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
    uint4* dst = reinterpret_cast<uint4*>(y + row * 128 + lane8 * 16);
    dst[0] = pack8(lo, unused);
    dst[1] = pack8(hi, unused);
  }
}

// ---- gated residual ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) gate_residual_kernel(uint4* __restrict__ x, const uint4* __restrict__ gate,
                                                            const uint4* __restrict__ y, long long vecs, int hidden_vecs,
                                                            int rows_per_batch) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / hidden_vecs;
    const int c = (int)(i - row * hidden_vecs);
    float a[8], g[8], b[8], r[8], unused = 0.f;
    unpack8(x[i], a);
    unpack8(__ldg(gate + (row / rows_per_batch) * hidden_vecs + c), g);
    unpack8(__ldg(y + i), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = __fmaf_rn(g[j], b[j], a[j]);
    x[i] = pack8(r, unused);
  }
}

int grid_for(long long vecs) {
  const long long want = (vecs + 255) / 256;
  return (int)(want < 148 * 16 ? (want > 0 ? want : 1) : 148 * 16);
}
bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

}  // namespace

extern "C" int tw_activate(const void* a, const void* b, void* y, float* stats, void* scratch, long long n, int mode,
                           void* stream_) {
  if (!a || !y || n <= 0 || (mode == TW_ACT_MUL && !b) || (stats && !scratch)) return TW_ERR_ARGUMENT;
  if (mode != TW_ACT_RELU2 && mode != TW_ACT_MUL && mode != TW_ACT_GELU_TANH) return TW_ERR_ARGUMENT;
  if (n % 8) return TW_ERR_SHAPE;
  if (misaligned(a) || misaligned(y) || (b && misaligned(b))) return TW_ERR_ALIGNMENT;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long vecs = n / 8;
  const int grid = grid_for(vecs);
  auto A = static_cast<const uint4*>(a), B = static_cast<const uint4*>(b);
  auto Y = static_cast<uint4*>(y);
  auto S = static_cast<unsigned*>(scratch);
  if (mode == TW_ACT_RELU2) activate_kernel<TW_ACT_RELU2><<<grid, 256, 0, stream>>>(A, B, Y, vecs, S, stats);
  else if (mode == TW_ACT_MUL) activate_kernel<TW_ACT_MUL><<<grid, 256, 0, stream>>>(A, B, Y, vecs, S, stats);
  else activate_kernel<TW_ACT_GELU_TANH><<<grid, 256, 0, stream>>>(A, B, Y, vecs, S, stats);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

extern "C" int tw_rms_norm(const void* x, const void* weight, const void* shift, const void* scale, void* y, float* stats,
                           void* scratch, int rows, int hidden, int rows_per_batch, float eps, void* stream_) {
  if (!x || !y || rows <= 0 || hidden <= 0 || rows_per_batch <= 0 || (stats && !scratch) || (!shift != !scale)) return TW_ERR_ARGUMENT;
  if (hidden % 8) return TW_ERR_SHAPE;
  if (hidden > 8 * 256 * 8) return TW_ERR_TOO_LARGE;
  if (misaligned(x) || misaligned(y) || (weight && misaligned(weight)) || (shift && (misaligned(shift) || misaligned(scale))))
    return TW_ERR_ALIGNMENT;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int hv = hidden / 8, vpt = (hv + 255) / 256;
  auto X = static_cast<const uint4*>(x), W = static_cast<const uint4*>(weight), SH = static_cast<const uint4*>(shift),
       SC = static_cast<const uint4*>(scale);
  auto Y = static_cast<uint4*>(y);
  auto S = static_cast<unsigned*>(scratch);
  if (vpt <= 1) rms_norm_kernel<1><<<rows, 256, 0, stream>>>(X, W, SH, SC, Y, hv, rows_per_batch, eps, S, stats);
  else if (vpt <= 2) rms_norm_kernel<2><<<rows, 256, 0, stream>>>(X, W, SH, SC, Y, hv, rows_per_batch, eps, S, stats);
  else if (vpt <= 4) rms_norm_kernel<4><<<rows, 256, 0, stream>>>(X, W, SH, SC, Y, hv, rows_per_batch, eps, S, stats);
  else rms_norm_kernel<8><<<rows, 256, 0, stream>>>(X, W, SH, SC, Y, hv, rows_per_batch, eps, S, stats);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

extern "C" int tw_rms_norm_heads(const void* x, void* y, long long tokens, int heads, long long stride_token,
                                 long long stride_head, float eps, void* stream_) {
  if (!x || !y || tokens <= 0 || heads <= 0) return TW_ERR_ARGUMENT;
  if (misaligned(x) || misaligned(y) || ((stride_token | stride_head) & 7)) return TW_ERR_ALIGNMENT;
  const long long rows = tokens * heads;
  head_rows_kernel<true, false, float><<<(unsigned)((rows + 31) / 32), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), rows, heads, stride_token, stride_head, eps,
      nullptr, nullptr, 1);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

extern "C" int tw_rope_heads(const void* x, void* y, long long tokens, int heads, long long stride_token, long long stride_head,
                             const void* cos_table, const void* sin_table, long long table_rows, int table_is_bf16, int norm,
                             float eps, void* stream_) {
  if (!x || !y || !cos_table || !sin_table || tokens <= 0 || heads <= 0 || table_rows <= 0) return TW_ERR_ARGUMENT;
  if (misaligned(x) || misaligned(y) || misaligned(cos_table) || misaligned(sin_table) || ((stride_token | stride_head) & 7))
    return TW_ERR_ALIGNMENT;
  const long long rows = tokens * heads;
  const unsigned grid = (unsigned)((rows + 31) / 32);
  cudaStream_t st = static_cast<cudaStream_t>(stream_);
  const __nv_bfloat16* xi = static_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* yo = static_cast<__nv_bfloat16*>(y);
  if (table_is_bf16) {
    const __nv_bfloat16 *c = static_cast<const __nv_bfloat16*>(cos_table), *sn = static_cast<const __nv_bfloat16*>(sin_table);
    if (norm) head_rows_kernel<true, true, __nv_bfloat16><<<grid, 256, 0, st>>>(xi, yo, rows, heads, stride_token, stride_head, eps, c, sn, table_rows);
    else head_rows_kernel<false, true, __nv_bfloat16><<<grid, 256, 0, st>>>(xi, yo, rows, heads, stride_token, stride_head, eps, c, sn, table_rows);
  } else {
    const float *c = static_cast<const float*>(cos_table), *sn = static_cast<const float*>(sin_table);
    if (norm) head_rows_kernel<true, true, float><<<grid, 256, 0, st>>>(xi, yo, rows, heads, stride_token, stride_head, eps, c, sn, table_rows);
    else head_rows_kernel<false, true, float><<<grid, 256, 0, st>>>(xi, yo, rows, heads, stride_token, stride_head, eps, c, sn, table_rows);
  }
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

extern "C" int tw_gate_residual(void* x, const void* gate, const void* y, int rows, int hidden, int rows_per_batch,
                                void* stream_) {
  if (!x || !gate || !y || rows <= 0 || hidden <= 0 || rows_per_batch <= 0) return TW_ERR_ARGUMENT;
  if (hidden % 8) return TW_ERR_SHAPE;
  if (misaligned(x) || misaligned(gate) || misaligned(y)) return TW_ERR_ALIGNMENT;
  const long long vecs = (long long)rows * (hidden / 8);
  gate_residual_kernel<<<grid_for(vecs), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<uint4*>(x), static_cast<const uint4*>(gate), static_cast<const uint4*>(y), vecs, hidden / 8, rows_per_batch);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}
