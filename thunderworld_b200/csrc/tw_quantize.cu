// Activation quantizer: bf16 [M,K] -> NVFP4 base plane A0 and residual plane A1 = A - deq(A0),
// both as E2M1 codes + E4M3 per-16 scales under one fp32 tensor factor, with the block scales
// written row-major (parity artefact, consumed by nothing on the GPU) and in the 128x4 atom layout
// the block-scaled MMA reads. Arithmetic follows the reference encoder operation by operation
// (thunderworld_fp4/cosmos/calibration.py:30-54, _quantize.py:81-107, _calibrated.py:11-38):
// IEEE fp32 division, E4M3 and E2M1 round-to-nearest-even, residual taken from the rounded base.
#include <type_traits>
#include <atomic>
#include "tw_common.cuh"
#include "../../include/twb200.h"

namespace {

constexpr int TILE = 128;          // rows and columns of one CTA tile (the repair lattice)
constexpr int PACK_THREADS = 256;  // 32 rows x 8 groups of 16 per pass, 4 passes

struct PackParams {
  const __nv_bfloat16* x;
  const float* prescale;
  const float* sensitivity;
  float* factor;
  const float* wg;
  float* alpha;
  uint8_t* codes;
  uint8_t* scales;
  uint8_t* scales_swz;
  int swz_rows;             // rows per plane of scales_swz
  const uint8_t* mask;
  const unsigned* amax_bits;
  float* scores;
  int m, k, mp, mb;
  int repair, factor_given;
  float base, res, gain;
};

__device__ __forceinline__ float load_factor(const PackParams& p) {
  if (p.factor_given) return *p.factor;
  float peak = __uint_as_float(*p.amax_bits);
  return peak > 0.f ? __fdiv_rn(peak, 2688.f) : 1.f;
}

// max |bf16(x * d)| over the tensor, as the bit pattern of a non-negative float. Each thread keeps four
// 16-byte loads in flight; without a prescale the maximum is taken on packed bf16 pairs (the maximum of
// bf16 magnitudes is a bf16 value, so nothing is rounded).
template <bool PRESCALE>
__global__ void __launch_bounds__(256) amax_kernel(const uint4* __restrict__ x, const float* __restrict__ d,
                                                   long long vecs, int k, unsigned* __restrict__ out) {
  float peak = 0.f;
  __nv_bfloat162 pk = __floats2bfloat162_rn(0.f, 0.f);
  for (long long base = (long long)blockIdx.x * 1024; base < vecs; base += (long long)gridDim.x * 1024) {
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long i = base + j * 256 + threadIdx.x;
      v[j] = i < vecs ? __ldg(x + i) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t w[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
      if (PRESCALE) {
        const long long i = base + j * 256 + threadIdx.x;
        const int col = (int)((i * 8) % k);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float lo = tw::bf16_bits_to_float(w[q] & 0xffffu), hi = tw::bf16_bits_to_float(w[q] >> 16);
          lo = __bfloat162float(__float2bfloat16_rn(__fmul_rn(lo, __ldg(d + col + 2 * q))));
          hi = __bfloat162float(__float2bfloat16_rn(__fmul_rn(hi, __ldg(d + col + 2 * q + 1))));
          peak = fmaxf(peak, fmaxf(fabsf(lo), fabsf(hi)));
        }
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) pk = __hmax2(pk, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[q])));
      }
    }
  }
  if (!PRESCALE) peak = fmaxf(__low2float(pk), __high2float(pk));
#pragma unroll
  for (int o = 16; o; o >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
  // one atomic per CTA: thousands of warps updating one word serialise in the L2
  __shared__ float warp_peak[8];
  if ((threadIdx.x & 31) == 0) warp_peak[threadIdx.x >> 5] = peak;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < 8; ++w) peak = fmaxf(peak, warp_peak[w]);
    if (peak > 0.f) atomicMax(out, __float_as_uint(peak));
  }
}

// Correctly rounded a / b from r = RN(1 / b): q0 = RN(a r), e = a - b q0 (exact in an FMA),
// q = RN(q0 + e r). For every divisor that is an E4M3 value this equals IEEE division for all
// float32 numerators (tests/exact_division_check.c enumerates every mantissa pair); for the tensor
// factor the kernel checks the 128 possible bf16 numerator mantissas itself before relying on it.
// The sign of a zero numerator is restored (the FMA chain turns -0 into +0).
__device__ __forceinline__ float div_by(float a, float b, float r) {
  float q0 = __fmul_rn(a, r);
  float e = __fmaf_rn(-b, q0, a);
  float q = __fmaf_rn(e, r, q0);
  return __uint_as_float(__float_as_uint(q) | (__float_as_uint(a) & 0x80000000u));
}
// Two quotients per instruction (fma.rn.f32x2 of sm_100): same three-operation sequence, without the
// sign fix; `nb` = -b. Callers restore the sign of zero where it is observable (the E2M1 code of -0).
__device__ __forceinline__ float2 div_by2(float2 a, float nb, float r) {
  const float2 r2 = make_float2(r, r);
  const float2 q0 = __fmul2_rn(a, r2);
  const float2 e = __ffma2_rn(make_float2(nb, nb), q0, a);
  return __ffma2_rn(e, r2, q0);
}
__device__ __forceinline__ float with_sign_of(float q, float a) {
  return __uint_as_float(__float_as_uint(q) | (__float_as_uint(a) & 0x80000000u));
}
// four code bytes (one per register, upper bits clear) -> one word, first byte lowest
__device__ __forceinline__ uint32_t pack4(uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
  return __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
}
// The two values of one code byte (low nibble first) as floats, exact.
__device__ __forceinline__ float2 e2m1x2_values(uint32_t byte) {
  uint32_t h2;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "r"(byte));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}

__device__ __forceinline__ uint32_t scale_offset(int row, int col, int cols) {
  return (uint32_t)(row >> 7) * 128u * cols + (uint32_t)(col >> 2) * 512u + (uint32_t)(row & 31) * 16u +
         (uint32_t)((row & 127) >> 5) * 4u + (uint32_t)(col & 3);
}

// Same for eight value pairs. `sign` (optional) supplies the sign of zero quotients: sign[i] has the sign
// the i-th pair's codes must carry (the pre-division values, whose -0 the packed division lost).
template <bool FAST, bool SIGN>
__device__ __forceinline__ uint32_t encode_group2(const float2 (&z)[8], const float2 (&sign)[8], float multiplier,
                                                  uint32_t (&bytes)[8], float& scale_value) {
  float peak = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) peak = fmaxf(peak, fmaxf(fabsf(z[i].x), fabsf(z[i].y)));
  float raw = __fdiv_rn(__fmul_rn(peak, multiplier), 6.f);
  raw = fminf(fmaxf(raw, 0.001953125f), 448.f);
  const uint32_t sb = tw::f32_to_e4m3(raw);
  const float s = tw::e4m3_to_f32(sb);
  const float rs = __frcp_rn(s);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float2 q;
    if (FAST) q = div_by2(z[i], -s, rs);
    else q = make_float2(__fdiv_rn(z[i].x, s), __fdiv_rn(z[i].y, s));
    if (SIGN) { q.x = with_sign_of(q.x, sign[i].x); q.y = with_sign_of(q.y, sign[i].y); }
    bytes[i] = tw::f32x2_to_e2m1x2(q.x, q.y);
  }
  scale_value = s;
  return sb;
}

// May the reciprocal sequence replace IEEE division by f? Every bf16 numerator mantissa is tried (one per thread
// of the first four warps); CTA-wide vote.
__device__ __forceinline__ bool fast_division_ok(float f, float rf) {
  int fast_ok = f > 8.6736174e-19f && f < 1.1529215e18f;        // 2^-60 .. 2^60: no under/overflow inside
  const float a = __uint_as_float(0x3f800000u | ((uint32_t)(threadIdx.x & 127) << 16));   // every group of 128 threads tries them all
  fast_ok = fast_ok && (div_by(a, f, rf) == __fdiv_rn(a, f));
  return __syncthreads_and(fast_ok) != 0;
}

// One 128x128 tile of the lattice, packed by the 256 threads of a CTA from `raw` (this thread's 16 consecutive
// bf16 values of rows pass*32 + r0, pass = 0..3, wherever they were staged).
template <bool PRESCALE, int REPAIR>
__device__ __forceinline__ void pack_tile(const PackParams& p, int kb, int mbi, float f, float rf, bool fast,
                                          const uint4 (&raw)[4][2], float* warp_scores, int group = 0) {
  const int t = threadIdx.x & (PACK_THREADS - 1), cg = t & 7, r0 = t >> 3;
  const int col = kb * TILE + cg * 16;
  const int kbn = p.k / TILE;
  const int cols16 = p.k / 16;
  constexpr bool planes2 = REPAIR != 0;
  const bool active = REPAIR != 2 || p.mask[mbi * kbn + kb] != 0;
  float dsc[16], sens[16];
  if (PRESCALE) {
#pragma unroll
    for (int i = 0; i < 16; ++i) dsc[i] = __ldg(p.prescale + col + i);
  }
  if (REPAIR == 3) {
#pragma unroll
    for (int i = 0; i < 16; ++i) sens[i] = __ldg(p.sensitivity + col + i);
  }
  float2 score2 = make_float2(0.f, 0.f);
  auto run = [&](auto fast_tag) {
  constexpr bool FAST = decltype(fast_tag)::value;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int row = mbi * TILE + pass * 32 + r0;
    float y[16];
    {
      const uint4 a = raw[pass][0], b = raw[pass][1];
      uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        y[2 * i] = tw::bf16_bits_to_float(w[i] & 0xffffu);
        y[2 * i + 1] = tw::bf16_bits_to_float(w[i] >> 16);
      }
      if (PRESCALE) {
#pragma unroll
        for (int i = 0; i < 16; ++i) y[i] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(y[i], dsc[i])));
      }
    }
    // z = y / f, two per instruction; the sign of a zero is carried by y
    float2 y2[8], z2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      y2[i] = make_float2(y[2 * i], y[2 * i + 1]);
      z2[i] = FAST ? div_by2(y2[i], -f, rf) : make_float2(__fdiv_rn(y[2 * i], f), __fdiv_rn(y[2 * i + 1], f));
    }
    uint2 c0, c1 = make_uint2(0u, 0u);
    float s0, s1;
    uint32_t b0[8];
    uint32_t sb0 = encode_group2<FAST, true>(z2, y2, p.base, b0, s0), sb1 = 0u;
    c0 = make_uint2(pack4(b0[0], b0[1], b0[2], b0[3]), pack4(b0[4], b0[5], b0[6], b0[7]));
    if (planes2) {
      float2 r2[8];
      const float2 ns0 = make_float2(-s0, -s0);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        // the product value * scale is exact in float32, so one FMA equals multiply-then-subtract
        r2[i] = __ffma2_rn(e2m1x2_values(b0[i]), ns0, z2[i]);
        if (REPAIR == 3) {
          // selector energy in the normalised domain: sum r^2 * sens (the common factor f^2 of the
          // unnormalised residual does not change the ranking or the energy-prefix ratio)
          score2 = __ffma2_rn(__fmul2_rn(r2[i], r2[i]), make_float2(sens[2 * i], sens[2 * i + 1]), score2);
        }
      }
      if (active) {
        uint32_t b1[8];
        sb1 = encode_group2<FAST, false>(r2, r2, p.res, b1, s1);
        c1 = make_uint2(pack4(b1[0], b1[1], b1[2], b1[3]), pack4(b1[4], b1[5], b1[6], b1[7]));
        if (p.gain != 1.f) sb1 = tw::f32_to_e4m3(fminf(__fmul_rn(s1, p.gain), 448.f));
      }
    }
    if (row >= p.mp) { sb0 = 0u; sb1 = 0u; }
    // gather the 8 scale bytes of this row's K128 block into lanes cg == 0 (all) and cg == 4 (upper half)
    uint32_t lo0 = sb0, lo1 = sb1;
#pragma unroll
    for (int j = 1; j < 4; ++j) {
      lo0 |= __shfl_down_sync(0xffffffffu, sb0, j) << (8 * j);
      lo1 |= __shfl_down_sync(0xffffffffu, sb1, j) << (8 * j);
    }
    uint32_t hi0 = __shfl_down_sync(0xffffffffu, lo0, 4), hi1 = __shfl_down_sync(0xffffffffu, lo1, 4);
    if (row < p.mp) {
      size_t ci = (size_t)row * (p.k / 2) + kb * 64 + cg * 8;
      *reinterpret_cast<uint2*>(p.codes + ci) = c0;
      if (planes2) *reinterpret_cast<uint2*>(p.codes + (size_t)p.mp * (p.k / 2) + ci) = c1;
      if (cg == 0) {
        size_t si = (size_t)row * cols16 + kb * 8;
        *reinterpret_cast<uint2*>(p.scales + si) = make_uint2(lo0, hi0);
        if (planes2) *reinterpret_cast<uint2*>(p.scales + (size_t)p.mp * cols16 + si) = make_uint2(lo1, hi1);
      }
    }
    if (p.scales_swz && (cg & 3) == 0) {
      uint32_t off = scale_offset(row, kb * 8 + cg, cols16);
      *reinterpret_cast<uint32_t*>(p.scales_swz + off) = lo0;
      if (planes2) *reinterpret_cast<uint32_t*>(p.scales_swz + (size_t)p.swz_rows * cols16 + off) = lo1;
    }
  }
  };
  if (fast) run(std::true_type{}); else run(std::false_type{});
  if (REPAIR == 3) {
    float score = __fadd_rn(score2.x, score2.y);
#pragma unroll
    for (int o = 16; o; o >>= 1) score = __fadd_rn(score, __shfl_xor_sync(0xffffffffu, score, o));
    // barriers of the 256 threads that pack this tile (a CTA may hold several such groups)
    if ((t & 31) == 0) warp_scores[t >> 5] = score;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "n"(PACK_THREADS) : "memory");
    if (t == 0) {
      float total = 0.f;
      for (int w = 0; w < PACK_THREADS / 32; ++w) total = __fadd_rn(total, warp_scores[w]);
      p.scores[mbi * kbn + kb] = total;
    }
    asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "n"(PACK_THREADS) : "memory");   // warp_scores is reused by the next tile
  }
}

// This thread's share of tile (mbi, kb): four rows, 32 bytes each; rows beyond m read as zeros.
__device__ __forceinline__ void load_tile_rows(const PackParams& p, int kb, int mbi, uint4 (&raw)[4][2]) {
  const int t = threadIdx.x & (PACK_THREADS - 1), cg = t & 7, r0 = t >> 3;
  const int col = kb * TILE + cg * 16;
#pragma unroll
  for (int pass = 0; pass < 4; ++pass) {
    const int row = mbi * TILE + pass * 32 + r0;
    if (row < p.m) {
      const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)row * p.k + col);
      raw[pass][0] = __ldg(src);
      raw[pass][1] = __ldg(src + 1);
    } else {
      raw[pass][0] = raw[pass][1] = make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

__device__ __forceinline__ void publish_factor(const PackParams& p, float f) {
  if (!p.factor_given) *p.factor = f;
  if (p.alpha && p.wg) *p.alpha = __fmul_rn(f, *p.wg);
}

// Two-launch form (the factor comes from amax_kernel or from the producer of x):
// grid (K/128, ceil(M/128)); each CTA packs one 128x128 tile of the lattice.
template <bool PRESCALE, int REPAIR>
__global__ void __launch_bounds__(PACK_THREADS, 3) pack_kernel(PackParams p) {
  __shared__ float warp_scores[PACK_THREADS / 32];
  const int kb = blockIdx.x, mbi = blockIdx.y;
  const float f = load_factor(p);
  const float rf = __frcp_rn(f);
  const bool fast = fast_division_ok(f, rf);
  // all four passes' loads are issued before any arithmetic so that 128 bytes per thread are in flight
  uint4 raw[4][2];
  load_tile_rows(p, kb, mbi, raw);
  pack_tile<PRESCALE, REPAIR>(p, kb, mbi, f, rf, fast, raw, warp_scores);
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) publish_factor(p, f);
}

// Single-pass form: x is read from global memory once. A cooperative grid of resident CTAs (one per SM) parks
// its tiles in shared memory while it reduces max|bf16(x d)|, meets at a grid barrier, and packs from shared
// memory under the tensor factor. Used when the tensor fits (tiles <= RESIDENT_TILES per CTA) and the caller
// gives no factor. The barrier wait is bounded: on a timeout (it cannot happen under a cooperative launch, which
// guarantees that every CTA is resident) the status word is set and the CTA returns.
constexpr int RESIDENT_TILES = 7;                        // 7 x 32 KB of the 227 KB a CTA may hold
constexpr int RESIDENT_GROUPS = 2;                       // groups of PACK_THREADS threads, each packs one tile at a time
template <bool PRESCALE, int REPAIR>
__global__ void __launch_bounds__(RESIDENT_GROUPS * PACK_THREADS, 1) pack_resident_kernel(PackParams p, int tiles, unsigned* header) {
  extern __shared__ uint4 slab[];                        // [tile slot][pass][256 threads][2]
  __shared__ float warp_scores[RESIDENT_GROUPS][PACK_THREADS / 32];
  __shared__ float warp_peak[RESIDENT_GROUPS * PACK_THREADS / 32];
  __shared__ int give_up;
  const int t = threadIdx.x & (PACK_THREADS - 1), group = threadIdx.x / PACK_THREADS;
  const int kbn = p.k / TILE;
  float peak = 0.f;
  __nv_bfloat162 pk = __floats2bfloat162_rn(0.f, 0.f);
  // this CTA's tiles are blockIdx.x, + gridDim.x, ...; its groups take them alternately; slot = position in the CTA
  int slot = group;
  for (int tile = blockIdx.x + group * gridDim.x; tile < tiles; tile += RESIDENT_GROUPS * gridDim.x, slot += RESIDENT_GROUPS) {
    const int mbi = tile / kbn, kb = tile % kbn;
    uint4 raw[4][2];
    load_tile_rows(p, kb, mbi, raw);
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        slab[((slot * 4 + pass) * 2 + j) * PACK_THREADS + t] = raw[pass][j];
        const uint32_t w[4] = {raw[pass][j].x, raw[pass][j].y, raw[pass][j].z, raw[pass][j].w};
        if (PRESCALE) {
          const float* d = p.prescale + kb * TILE + (t & 7) * 16 + j * 8;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float lo = tw::bf16_bits_to_float(w[q] & 0xffffu), hi = tw::bf16_bits_to_float(w[q] >> 16);
            lo = __bfloat162float(__float2bfloat16_rn(__fmul_rn(lo, __ldg(d + 2 * q))));
            hi = __bfloat162float(__float2bfloat16_rn(__fmul_rn(hi, __ldg(d + 2 * q + 1))));
            peak = fmaxf(peak, fmaxf(fabsf(lo), fabsf(hi)));
          }
        } else {
#pragma unroll
          for (int q = 0; q < 4; ++q) pk = __hmax2(pk, __habs2(*reinterpret_cast<const __nv_bfloat162*>(&w[q])));
        }
      }
    }
  }
  if (!PRESCALE) peak = fmaxf(__low2float(pk), __high2float(pk));
#pragma unroll
  for (int o = 16; o; o >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
  if ((threadIdx.x & 31) == 0) warp_peak[threadIdx.x >> 5] = peak;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int w = 1; w < RESIDENT_GROUPS * PACK_THREADS / 32; ++w) peak = fmaxf(peak, warp_peak[w]);
    if (peak > 0.f) atomicMax(header, __float_as_uint(peak));
    __threadfence();
    atomicAdd(header + 1, 1u);
    // grid barrier, bounded
    int bad = 0;
    const long long start = clock64();
    while (atomicAdd(header + 1, 0u) < gridDim.x) {
      __nanosleep(40);
      if (clock64() - start > 1000000000LL) { bad = 1; atomicExch(header + 2, (unsigned)TW_ERR_TIMEOUT); break; }
    }
    __threadfence();
    give_up = bad;
  }
  __syncthreads();
  if (give_up) return;
  const float f = load_factor(p);
  const float rf = __frcp_rn(f);
  const bool fast = fast_division_ok(f, rf);
  slot = group;
  for (int tile = blockIdx.x + group * gridDim.x; tile < tiles; tile += RESIDENT_GROUPS * gridDim.x, slot += RESIDENT_GROUPS) {
    const int mbi = tile / kbn, kb = tile % kbn;
    uint4 raw[4][2];
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
      raw[pass][0] = slab[((slot * 4 + pass) * 2 + 0) * PACK_THREADS + t];
      raw[pass][1] = slab[((slot * 4 + pass) * 2 + 1) * PACK_THREADS + t];
    }
    pack_tile<PRESCALE, REPAIR>(p, kb, mbi, f, rf, fast, raw, warp_scores[group], group);
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) publish_factor(p, f);
}

// Per M128 row block: rank K128 blocks by score (descending, lower index wins ties), keep rank < na,
// optionally stop at the shortest prefix holding `energy` of the total (_sparse_pack.py:46-61).
__global__ void __launch_bounds__(128) choose_kernel(const float* __restrict__ scores, uint8_t* __restrict__ mask,
                                                     int kbn, int na, float energy) {
  extern __shared__ float row[];
  const int mb = blockIdx.x;
  for (int j = threadIdx.x; j < kbn; j += blockDim.x) row[j] = scores[mb * kbn + j];
  __syncthreads();
  float total = 0.f;
  if (energy < 1.f)
    for (int j = 0; j < kbn; ++j) total = __fadd_rn(total, row[j]);
  for (int j = threadIdx.x; j < kbn; j += blockDim.x) {
    const float mine = row[j];
    int rank = 0;
    for (int o = 0; o < kbn; ++o) rank += (row[o] > mine) || (row[o] == mine && o < j);
    bool keep = rank < na;
    if (keep && energy < 1.f) {
      float before = 0.f;
      for (int o = 0; o < kbn; ++o)
        if ((row[o] > mine) || (row[o] == mine && o < j)) before = __fadd_rn(before, row[o]);
      keep = before < __fmul_rn(energy, total);
    }
    mask[mb * kbn + j] = keep ? 1 : 0;
  }
}

// Sampled-energy rank of every K128 block within its M128 row block (reference: activation_rank,
// thunderworld_fp4/_linear_kernels.py:23-34): eight rows (every 16th, clamped to the last row) and eight columns
// (every 16th) of bf16(x * d) per 128x128 block; rank 0 = largest energy, the lower index wins ties.
__global__ void __launch_bounds__(128) rank_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ d,
                                                   int m, int k, int* __restrict__ rank) {
  extern __shared__ float energy[];
  const int mb = blockIdx.x, kbn = k / TILE;
  for (int kb = threadIdx.x; kb < kbn; kb += blockDim.x) {
    float e = 0.f;
    for (int i = 0; i < 8; ++i) {
      const int row = min(mb * TILE + i * 16, m - 1);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int col = kb * TILE + j * 16;
        float v = __bfloat162float(x[(size_t)row * k + col]);
        if (d) v = __bfloat162float(__float2bfloat16_rn(__fmul_rn(v, __ldg(d + col))));
        e = __fmaf_rn(v, v, e);
      }
    }
    energy[kb] = e;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < kbn; j += blockDim.x) {
    const float mine = energy[j];
    int r = 0;
    for (int o = 0; o < kbn; ++o) r += (energy[o] > mine) || (energy[o] == mine && o < j);
    rank[mb * kbn + j] = r;
  }
}

__global__ void __launch_bounds__(256) swizzle_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                                      int rows, int cols, int rows_padded) {
  // one thread per 4 consecutive scale columns of one row
  const int quads = cols >> 2;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= (long long)rows_padded * quads) return;
  int row = (int)(i / quads), q = (int)(i % quads);
  uint32_t v = row < rows ? *reinterpret_cast<const uint32_t*>(src + (size_t)row * cols + q * 4) : 0u;
  *reinterpret_cast<uint32_t*>(dst + scale_offset(row, q * 4, cols)) = v;
}

}  // namespace

extern "C" size_t tw_quantize_workspace(int m, int k) {
  if (m <= 0 || k <= 0) return 0;
  size_t mb = (size_t)(m + 127) / 128, kb = (size_t)(k + 127) / 128;
  return 256 + mb * kb * sizeof(float);
}

extern "C" int tw_quantize(const TwQuantizeArgs* a, void* stream_) {
  if (!a || !a->x || !a->codes || !a->scales || !a->factor || !a->workspace) return TW_ERR_ARGUMENT;
  if (a->m <= 0 || a->k <= 0) return TW_ERR_ARGUMENT;
  if (a->k % 128 || a->mp < (a->m + 15) / 16 * 16 || a->mp % 16) return TW_ERR_SHAPE;
  if (a->swz_rows && (a->swz_rows % 128 || a->swz_rows < (a->m + 127) / 128 * 128)) return TW_ERR_SHAPE;
  if (a->repair < 0 || a->repair > 3) return TW_ERR_ARGUMENT;
  if ((a->repair == 2 || a->repair == 3) && !a->mask) return TW_ERR_ARGUMENT;
  if (a->repair == 3 && (!a->sensitivity || a->na <= 0 || a->na >= a->k / 128)) return TW_ERR_ARGUMENT;
  if (!(a->base > 0.f) || !(a->res > 0.f) || !(a->gain > 0.f)) return TW_ERR_ARGUMENT;
  const uintptr_t align = (uintptr_t)a->x | (uintptr_t)a->codes | (uintptr_t)a->scales |
                          (uintptr_t)a->scales_swz | (uintptr_t)a->workspace;
  if (align & 15) return TW_ERR_ALIGNMENT;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  unsigned* amax = static_cast<unsigned*>(a->workspace);
  float* scores = reinterpret_cast<float*>(static_cast<char*>(a->workspace) + 256);
  const int mb = (a->m + 127) / 128, kb = a->k / 128;
  PackParams p{};
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.prescale = a->prescale; p.sensitivity = a->sensitivity;
  p.factor = a->factor; p.wg = a->wg; p.alpha = a->alpha;
  p.codes = a->codes; p.scales = a->scales; p.scales_swz = a->scales_swz; p.mask = a->mask;
  p.amax_bits = amax; p.scores = scores;
  p.m = a->m; p.k = a->k; p.mp = a->mp; p.mb = mb;
  p.swz_rows = a->swz_rows ? a->swz_rows : mb * 128;
  p.repair = a->repair; p.factor_given = a->factor_given;
  p.base = a->base; p.res = a->res; p.gain = a->gain;
  int dev = 0, sms = 0, coop = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TW_ERR_LAUNCH;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  const long long tiles = (long long)mb * kb;
  // single pass when the tensor can stay in shared memory between the reduction and the packing
  const bool resident = !a->factor_given && coop && sms > 0 && tiles <= (long long)RESIDENT_TILES * sms;
  if (!a->factor_given && cudaMemsetAsync(amax, 0, 16, stream) != cudaSuccess) return TW_ERR_LAUNCH;
  if (!a->factor_given && !resident) {
    long long vecs = (long long)a->m * a->k / 8;
    int blocks = (int)((vecs + 1023) / 1024 < 148 * 8 ? (vecs + 1023) / 1024 : 148 * 8);
    if (a->prescale)
      amax_kernel<true><<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(a->x), a->prescale, vecs, a->k, amax);
    else
      amax_kernel<false><<<blocks, 256, 0, stream>>>(static_cast<const uint4*>(a->x), nullptr, vecs, a->k, amax);
  }
  dim3 grid(kb, mb);
  int status = TW_OK;
  auto launch = [&](auto pre, auto mode) {
    constexpr bool PRE = decltype(pre)::value;
    constexpr int MODE = decltype(mode)::value;
    if (!resident) {
      pack_kernel<PRE, MODE><<<grid, PACK_THREADS, 0, stream>>>(p);
      return;
    }
    const int ctas = tiles < sms ? (int)tiles : sms;
    const int per_cta = (int)((tiles + ctas - 1) / ctas);
    const int smem = per_cta * TILE * TILE * 2;
    static std::atomic<int> configured[64];                  // largest opt-in made so far on this device
    if (configured[dev].load(std::memory_order_acquire) < smem) {
      if (cudaFuncSetAttribute(pack_resident_kernel<PRE, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               RESIDENT_TILES * TILE * TILE * 2) != cudaSuccess) { status = TW_ERR_LAUNCH; return; }
      configured[dev].store(RESIDENT_TILES * TILE * TILE * 2, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas); cfg.blockDim = dim3(RESIDENT_GROUPS * PACK_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative; attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, pack_resident_kernel<PRE, MODE>, p, (int)tiles, amax) != cudaSuccess) status = TW_ERR_LAUNCH;
  };
  auto by_mode = [&](auto pre) {
    switch (a->repair) {
      case 0: launch(pre, std::integral_constant<int, 0>{}); break;
      case 1: launch(pre, std::integral_constant<int, 1>{}); break;
      case 2: launch(pre, std::integral_constant<int, 2>{}); break;
      default: launch(pre, std::integral_constant<int, 3>{}); break;
    }
  };
  if (a->prescale) by_mode(std::true_type{}); else by_mode(std::false_type{});
  if (status != TW_OK) return status;
  if (a->repair == 3) choose_kernel<<<mb, 128, kb * sizeof(float), stream>>>(scores, a->mask, kb, a->na, a->energy);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

extern "C" int tw_activation_rank(const void* x, const float* prescale, int m, int k, int32_t* rank, void* stream_) {
  if (!x || !rank || m <= 0 || k <= 0) return TW_ERR_ARGUMENT;
  if (k % 128) return TW_ERR_SHAPE;
  const int mb = (m + 127) / 128, kb = k / 128;
  rank_kernel<<<mb, 128, kb * sizeof(float), static_cast<cudaStream_t>(stream_)>>>(static_cast<const __nv_bfloat16*>(x), prescale, m, k, rank);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

extern "C" int tw_swizzle_scales(const uint8_t* src, int rows, int cols, uint8_t* dst, void* stream_) {
  if (!src || !dst || rows <= 0 || cols <= 0) return TW_ERR_ARGUMENT;
  if (cols % 4) return TW_ERR_SHAPE;
  if (((uintptr_t)src | (uintptr_t)dst) & 3) return TW_ERR_ALIGNMENT;
  const int rp = (rows + 127) / 128 * 128;
  long long work = (long long)rp * (cols / 4);
  swizzle_kernel<<<(unsigned)((work + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream_)>>>(src, dst, rows, cols, rp);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------------------------
// Quantizer entry point for callers that cannot allocate device memory
// ---------------------------------------------------------------------------------------------
// Some hosts of this library may not call cudaMalloc at the point where they quantize: a plugin
// that runs inside another framework's memory plan, a real-time loop that forbids allocation after
// start-up, code running while a pool is frozen. tw_quantize needs a few KB of scratch (the
// amax word and one selector score per 128x128 lattice tile); here that scratch is a fixed array
// in the library's own device image, so the caller passes inputs and outputs only.
//
// The array exists once per GPU that loads the library and stays until the process exits. Every
// call on a device shares it and it keeps the previous call's contents: the amax word is cleared
// at the start of each call and the scores are fully rewritten before they are read, but two calls
// that overlap on the same GPU (different streams) race on it. The array name below is only a
// host-side handle; the device address is looked up once per device with cudaGetSymbolAddress.
namespace {
constexpr int STATIC_TILES = 16384;                       // lattice tiles: ceil(m/128) * (k/128) <= 16384
static __device__ __align__(256) unsigned char g_quantize_scratch[256 + STATIC_TILES * sizeof(float)];
constexpr int MAX_DEVICES = 64;
std::atomic<void*> g_scratch_address[MAX_DEVICES];      // zero-initialised; host threads may race to fill a slot
}  // namespace

extern "C" int tw_quantize_static_max_tiles(void) { return STATIC_TILES; }

extern "C" int tw_quantize_static(const TwQuantizeArgs* a, void* stream) {
  if (!a) return TW_ERR_ARGUMENT;
  if (a->m <= 0 || a->k <= 0) return TW_ERR_ARGUMENT;
  if (a->k % 128) return TW_ERR_SHAPE;
  const long long tiles = (long long)((a->m + 127) / 128) * (a->k / 128);
  if (tiles > STATIC_TILES) return TW_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return TW_ERR_LAUNCH;
  void* ptr = g_scratch_address[dev].load(std::memory_order_acquire);
  if (!ptr) {
    // first call on this device (it is the current one): resolve the device address of the array
    if (cudaGetSymbolAddress(&ptr, g_quantize_scratch) != cudaSuccess || !ptr) return TW_ERR_LAUNCH;
    g_scratch_address[dev].store(ptr, std::memory_order_release);
  }
  TwQuantizeArgs local = *a;
  local.workspace = ptr;
  return tw_quantize(&local, stream);
}
