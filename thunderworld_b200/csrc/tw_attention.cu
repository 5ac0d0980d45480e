// Streaming FP4 attention for sm_100a: online Q/K/V packing, tile selection and the attention kernel.
//
// Reference (Triton): packages/fp4-repair/src/thunderworld_fp4/_kernels.py
//   pack_qk :12-25, pack_v :29-47, streaming_attention :51-124, select_tiles_head :191-215
// and the per-row-factor quantizer _quantize.py:7-39 (factor = max(|row|max / 1536, 1e-12)).
// Packing is redone for every call; nothing about old inputs is cached. P is quantized on chip.
#include <type_traits>
#include <cuda.h>
#include <atomic>
#include "tw_common.cuh"
#include "../../include/twb200.h"

namespace {

// a / b from r = RN(1/b); exact for every E4M3 divisor (tests/exact_division_check.c).
__device__ __forceinline__ float div_by(float a, float b, float r) {
  float q0 = __fmul_rn(a, r);
  float e = __fmaf_rn(-b, q0, a);
  float q = __fmaf_rn(e, r, q0);
  return __uint_as_float(__float_as_uint(q) | (__float_as_uint(a) & 0x80000000u));
}
__device__ __forceinline__ float2 e2m1x2_values(uint32_t byte) {
  uint32_t h2;
  asm("{ .reg .b8 t; cvt.u8.u32 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(h2) : "r"(byte));
  return __half22float2(*reinterpret_cast<__half2*>(&h2));
}
// Quantize 16 normalised values: E4M3 scale byte, 8 code bytes; returns the scale value.
__device__ __forceinline__ float encode16(const float (&z)[16], uint32_t& scale_byte, uint2& codes) {
  float peak = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) peak = fmaxf(peak, fabsf(z[i]));
  const float raw = fmaxf(__fdiv_rn(peak, 6.f), 0.001953125f);
  scale_byte = tw::f32_to_e4m3(raw);
  const float s = tw::e4m3_to_f32(scale_byte), rs = __frcp_rn(s);
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i)
    w[i >> 2] |= tw::f32x2_to_e2m1x2(div_by(z[2 * i], s, rs), div_by(z[2 * i + 1], s, rs)) << (8 * (i & 3));
  codes = make_uint2(w[0], w[1]);
  return s;
}
// 128x8 scale atom: byte offset of (row within the 128-row block, scale column 0..7)
__device__ __forceinline__ uint32_t atom_offset(int row, int col) {
  return (uint32_t)(col >> 2) * 512u + (uint32_t)(row & 31) * 16u + (uint32_t)((row & 127) >> 5) * 4u + (uint32_t)(col & 3);
}

struct RowPackParams {
  const __nv_bfloat16* x;   // [rows, heads, 128] with strides (elements)
  uint8_t* codes;           // [planes, heads * rows_padded, 64]
  uint8_t* scales;          // [planes, heads * rows_padded, 8] row-major
  uint8_t* scales_swz;      // [planes, heads, ceil(rows_padded/128), 1024] atom layout
  float* factors;           // [heads * rows_padded]
  float* energy;            // V only: [heads, tiles, 8]
  long long stride_row, stride_head;
  int rows, heads, rows_padded, blocks128, repair, need_energy;
};

// Shared tail of both packers: the 8 lanes of a row (16 values each) quantize and store one row.
// `row_out` indexes the packed row inside its head, `lane8` the group of 16.
__device__ __forceinline__ void quantize_row_group(const RowPackParams& p, float (&x)[16], int head, int row_out,
                                                   int lane8, bool store) {
  float peak = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) peak = fmaxf(peak, fabsf(x[i]));
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
  const float f = fmaxf(__fdiv_rn(peak, 1536.f), 1.0e-12f);
  float z[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) z[i] = __fdiv_rn(x[i], f);
  uint32_t sb0, sb1 = 0u;
  uint2 c0, c1 = make_uint2(0u, 0u);
  const float s0 = encode16(z, sb0, c0);
  if (p.repair) {
    float r[16];
    const uint32_t w[2] = {c0.x, c0.y};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 v = e2m1x2_values((w[i >> 2] >> (8 * (i & 3))) & 0xffu);
      r[2 * i] = __fmaf_rn(-v.x, s0, z[2 * i]);
      r[2 * i + 1] = __fmaf_rn(-v.y, s0, z[2 * i + 1]);
    }
    encode16(r, sb1, c1);
  }
  uint32_t lo0 = sb0, lo1 = sb1;
#pragma unroll
  for (int j = 1; j < 4; ++j) {
    lo0 |= __shfl_down_sync(0xffffffffu, sb0, j) << (8 * j);
    lo1 |= __shfl_down_sync(0xffffffffu, sb1, j) << (8 * j);
  }
  const uint32_t hi0 = __shfl_down_sync(0xffffffffu, lo0, 4), hi1 = __shfl_down_sync(0xffffffffu, lo1, 4);
  if (!store) return;
  const size_t row = (size_t)head * p.rows_padded + row_out;
  const size_t plane_rows = (size_t)p.heads * p.rows_padded;
  *reinterpret_cast<uint2*>(p.codes + row * 64 + lane8 * 8) = c0;
  if (p.repair) *reinterpret_cast<uint2*>(p.codes + (plane_rows + row) * 64 + lane8 * 8) = c1;
  const size_t atom = ((size_t)head * p.blocks128 + (row_out >> 7)) * 1024;
  const size_t plane_atoms = (size_t)p.heads * p.blocks128 * 1024;
  if (lane8 == 0) {
    *reinterpret_cast<uint2*>(p.scales + row * 8) = make_uint2(lo0, hi0);
    if (p.repair) *reinterpret_cast<uint2*>(p.scales + (plane_rows + row) * 8) = make_uint2(lo1, hi1);
    p.factors[row] = f;
  }
  if ((lane8 & 3) == 0) {
    *reinterpret_cast<uint32_t*>(p.scales_swz + atom + atom_offset(row_out, lane8)) = lo0;
    if (p.repair) *reinterpret_cast<uint32_t*>(p.scales_swz + plane_atoms + atom + atom_offset(row_out, lane8)) = lo1;
  }
}

// Q or K: one row per (token, head). grid (ceil(rows_padded/32), heads), 256 threads = 32 rows x 8 groups.
__global__ void __launch_bounds__(256) pack_qk_kernel(RowPackParams p) {
  const int lane8 = threadIdx.x & 7, head = blockIdx.y;
  const int row = blockIdx.x * 32 + (threadIdx.x >> 3);
  float x[16];
  if (row < p.rows) {
    const uint4* src = reinterpret_cast<const uint4*>(p.x + (size_t)row * p.stride_row + (size_t)head * p.stride_head + lane8 * 16);
    const uint4 a = __ldg(src), b = __ldg(src + 1);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      x[2 * i] = tw::bf16_bits_to_float(w[i] & 0xffffu);
      x[2 * i + 1] = tw::bf16_bits_to_float(w[i] >> 16);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = 0.f;
  }
  quantize_row_group(p, x, head, row, lane8, row < p.rows_padded);
}

// V: rows of the packed tensor are (kv head, key tile, channel d), columns the 128 tokens of the tile.
// grid (tiles, heads); the CTA stages the 128 x 128 tile in shared memory to transpose it.
__global__ void __launch_bounds__(256) pack_v_kernel(RowPackParams p) {
  __shared__ __nv_bfloat16 tile[128][130];
  __shared__ float energy_part[8][4];
  const int nt = blockIdx.x, head = blockIdx.y, t = threadIdx.x;
  for (int i = t; i < 128 * 16; i += 256) {            // 16-byte pieces: token i/16, channels (i%16)*8..
    const int tok = i >> 4, piece = i & 15, token = nt * 128 + tok;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (token < p.rows)
      v = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)token * p.stride_row + (size_t)head * p.stride_head + piece * 8));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tile[tok][piece * 8 + 2 * j] = __ushort_as_bfloat16((unsigned short)(w[j] & 0xffffu));
      tile[tok][piece * 8 + 2 * j + 1] = __ushort_as_bfloat16((unsigned short)(w[j] >> 16));
    }
  }
  __syncthreads();
  const int lane8 = t & 7;
#pragma unroll 1
  for (int pass = 0; pass < 4; ++pass) {
    const int d = pass * 32 + (t >> 3);
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) x[i] = __bfloat162float(tile[lane8 * 16 + i][d]);
    if (p.need_energy) {
      float e = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) e = __fmaf_rn(x[i], x[i], e);
      // 16 channels x 128 tokens = one energy group: lanes of two 16-row halves of this pass
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) e += __shfl_xor_sync(0xffffffffu, e, o);
      // a warp covers 4 channels; 4 warps (16 channels) form one group of the 8 per tile
      if ((t & 31) == 0) energy_part[pass * 2 + ((t >> 5) >> 2)][(t >> 5) & 3] = e;
    }
    quantize_row_group(p, x, head, nt * 128 + d, lane8, true);
  }
  if (p.need_energy) {
    __syncthreads();
    if (t < 8)
      p.energy[((size_t)head * gridDim.x + nt) * 8 + t] =
          (energy_part[t][0] + energy_part[t][1] + energy_part[t][2] + energy_part[t][3]) * (1.f / 16384.f);
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Tile selector (reference: select_tiles_head, _kernels.py:191-215)
// ---------------------------------------------------------------------------------------------
namespace {

struct SelectParams {
  const __nv_bfloat16 *q, *k;
  const float* energy;        // [hk, nt, 8]
  int* flags;                 // [hq, mt, nt]
  int* pvflags;               // optional
  const int* counts;          // [hq]
  const int* pvcounts;        // optional [hq]
  long long q_row, q_head, k_row, k_head;
  int m, n, hq, hk, nt, terms, pvterms;
};

// One CTA per (query head, M128 block): eight sampled queries against eight sampled keys of every key
// tile, softmax over all samples, mass per tile x sqrt(V energy), rank (lower index wins ties).
__global__ void __launch_bounds__(128) select_kernel(SelectParams p) {
  extern __shared__ float sm[];
  float* qs = sm;                         // [8][128]
  float* sim = qs + 8 * 128;              // [8][nt*8]
  float* score = sim + 8 * p.nt * 8;      // [nt]
  const int h = blockIdx.x, mt = blockIdx.y, kh = h / (p.hq / p.hk), t = threadIdx.x;
  const int samples = p.nt * 8;
  {                                         // eight sampled query rows: thread t loads 8 channels of row t / 16
    const int i = t >> 4, c = t & 15;
    const int row = min(mt * 128 + i * 16, p.m - 1);
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p.q + (size_t)row * p.q_row + (size_t)h * p.q_head) + c);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      qs[i * 128 + c * 8 + 2 * j] = tw::bf16_bits_to_float(w[j] & 0xffffu);
      qs[i * 128 + c * 8 + 2 * j + 1] = tw::bf16_bits_to_float(w[j] >> 16);
    }
  }
  __syncthreads();
  for (int s = t; s < samples; s += 128) {
    const int key = (s >> 3) * 128 + (s & 7) * 16;
    // one key row = 256 contiguous bytes: sixteen 16-byte loads; the products are accumulated in channel order
    const uint4* kp = reinterpret_cast<const uint4*>(p.k + (size_t)min(key, p.n - 1) * p.k_row + (size_t)kh * p.k_head);
    float acc[8] = {};
#pragma unroll 2
    for (int c = 0; c < 16; ++c) {
      const uint4 raw = __ldg(kp + c);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      float kv[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        kv[2 * j] = tw::bf16_bits_to_float(w[j] & 0xffffu);
        kv[2 * j + 1] = tw::bf16_bits_to_float(w[j] >> 16);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 qa = *reinterpret_cast<const float4*>(qs + i * 128 + c * 8);
        const float4 qb = *reinterpret_cast<const float4*>(qs + i * 128 + c * 8 + 4);
        float a = acc[i];
        a = __fmaf_rn(qa.x, kv[0], a); a = __fmaf_rn(qa.y, kv[1], a); a = __fmaf_rn(qa.z, kv[2], a); a = __fmaf_rn(qa.w, kv[3], a);
        a = __fmaf_rn(qb.x, kv[4], a); a = __fmaf_rn(qb.y, kv[5], a); a = __fmaf_rn(qb.z, kv[6], a); a = __fmaf_rn(qb.w, kv[7], a);
        acc[i] = a;
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) sim[i * samples + s] = key < p.n ? acc[i] * 0.08838834764831845f : -INFINITY;
  }
  __syncthreads();
  // softmax per sampled query: warp w normalises queries w and w + 4
  const int warp = t >> 5, lane = t & 31;
  for (int i = warp; i < 8; i += 4) {
    float mx = -INFINITY;
    for (int s = lane; s < samples; s += 32) mx = fmaxf(mx, sim[i * samples + s]);
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int s = lane; s < samples; s += 32) {
      const float e = __expf(sim[i * samples + s] - mx);
      sim[i * samples + s] = e;
      sum += e;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum;
    for (int s = lane; s < samples; s += 32) sim[i * samples + s] *= inv;
  }
  __syncthreads();
  for (int tile = t; tile < p.nt; tile += 128) {
    float mass = 0.f, e = 0.f;
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 8; ++j) mass += sim[i * samples + tile * 8 + j];
    for (int g = 0; g < 8; ++g) e += p.energy[((size_t)kh * p.nt + tile) * 8 + g];
    score[tile] = mass * 0.125f * sqrtf(e);
  }
  __syncthreads();
  const int count = p.counts[h], pvcount = p.pvcounts ? p.pvcounts[h] : 0;
  for (int tile = t; tile < p.nt; tile += 128) {
    const float mine = score[tile];
    int rank = 0;
    for (int o = 0; o < p.nt; ++o) rank += (score[o] > mine) || (score[o] == mine && o < tile);
    const size_t idx = ((size_t)h * gridDim.y + mt) * p.nt + tile;
    p.flags[idx] = rank < count ? p.terms : 1;
    if (p.pvflags) p.pvflags[idx] = rank < pvcount ? p.pvterms : 1;
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// Streaming attention kernel (reference: streaming_attention, _kernels.py:51-124)
// ---------------------------------------------------------------------------------------------
// One CTA per (128-query tile, query head). For every key tile of 128:
//   S = Q0 K0^T [+ Q1 K0^T + Q0 K1^T + Q1 K1^T where the tile is selected]      tcgen05, fp32 in TMEM
//   s = S * qf[m] * kf[n] / sqrt(128); online softmax in fp32 (one query row per thread)
//   P quantized on chip to NVFP4 (per-row factor max/1536, E4M3 per 16, E2M1; reciprocals approximate
//   as in the reference's quantize_fast), residual P1 only where the PV tile is selected
//   T = P0 V0 [+ P1 V0 + P0 V1 + P1 V1]                                          tcgen05, fp32 in TMEM
//   acc = acc * alpha + T * pf[m] * vf[d]
// Warps: 0 producer (TMA + bulk copies), 1 MMA issuer (scale copies smem -> TMEM, MMAs, commits),
// 4..11 softmax (two groups of four warps), 12..19 accumulate (row = TMEM lane). No cluster, no multicast.
namespace {

constexpr int ATT_TILE = 128 * 64;        // bytes of a 128 x 128 NVFP4 code tile
constexpr int ATT_SF = 1024;
constexpr int ATT_SLOTS = 3;
constexpr int ATT_THREADS = 640;       // 4 control warps, 8 softmax warps, 8 accumulate warps
// Register budgets per thread after the warpgroups rebalance. The launch allocates ATT_REGS_LAUNCH for each
// of the 20 warps; a warpgroup that asks for more than the others have released waits forever, so the
// sum is checked here.
constexpr int ATT_REGS_LAUNCH = 96, ATT_REGS_CONTROL = 56, ATT_REGS_SOFTMAX = 104, ATT_REGS_ACCUM = 104;
static_assert(4 * ATT_REGS_CONTROL + 8 * ATT_REGS_SOFTMAX + 8 * ATT_REGS_ACCUM <= 20 * ATT_REGS_LAUNCH, "register budgets exceed the launch allocation");
constexpr int ATT_NT_MAX = 1024;

struct AttParams {
  const uint8_t *sfq, *sfk, *sfv;          // atom-layout scales [planes, heads, blocks, 1024]
  const float *qf, *kf, *vf;               // factors
  const int *flags, *pvflags;              // [hq, mb, nt] or null
  __nv_bfloat16* out;                      // [m, hq, 128]
  int* status;
  int m, n, hq, hk, mp, np, mblk, nt;
  int repair, full, terms, pv_repair, pv_full, pv_terms;
};

struct AttSmem {
  static constexpr int OFF_Q = 0;                                   // Q0, Q1
  static constexpr int OFF_K = OFF_Q + 2 * ATT_TILE;                // slots x (K0, K1)
  static constexpr int OFF_V = OFF_K + ATT_SLOTS * 2 * ATT_TILE;
  static constexpr int OFF_P = OFF_V + ATT_SLOTS * 2 * ATT_TILE;    // 2 buffers x (P0, P1)
  static constexpr int OFF_SFQ = OFF_P + 2 * 2 * ATT_TILE;
  static constexpr int OFF_SFK = OFF_SFQ + 2 * ATT_SF;
  static constexpr int OFF_SFV = OFF_SFK + ATT_SLOTS * 2 * ATT_SF;
  static constexpr int OFF_SFP = OFF_SFV + ATT_SLOTS * 2 * ATT_SF;
  static constexpr int OFF_KF = OFF_SFP + 2 * 2 * ATT_SF;           // slots x 128 floats
  static constexpr int OFF_VF = OFF_KF + ATT_SLOTS * 512;
  static constexpr int OFF_SEL = OFF_VF + ATT_SLOTS * 512;          // per key tile: bit0 QK repair, bit1 PV repair
  static constexpr int OFF_STAT = (OFF_SEL + ATT_NT_MAX + 15) / 16 * 16;  // ring of 4 x 128 rows x (ref, pf, row sum, -)
  static constexpr int OFF_GMAX = OFF_STAT + 4 * 128 * 16;          // 2 softmax groups x 8 K16 groups x 128 rows: group maxima
  static constexpr int OFF_BAR = OFF_GMAX + 2 * 8 * 128 * 4;
  static constexpr int NUM_BARS = 1 + 4 * ATT_SLOTS + 2 + 2 + 2 + 2 + 2 + 2 + 4;
  static constexpr int BYTES = OFF_BAR + NUM_BARS * 8 + 64 + 1024;
};
// tensor-memory columns
constexpr int TM_S = 0, TM_T = 256, TM_SFQ0 = 384, TM_SFQ1 = 392, TM_SFK0 = 400, TM_SFK1 = 416, TM_SFP0 = 432,
              TM_SFP1 = 448, TM_SFV0 = 464, TM_SFV1 = 480;

__device__ __forceinline__ float rcp_approx(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float r;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float exp2_approx(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__global__ void __launch_bounds__(ATT_THREADS, 1)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttParams p) {
  using L = AttSmem;
  extern __shared__ uint8_t smem_raw[];
  // aligned by pointer arithmetic on the __shared__ array (not through an integer cast), so that the compiler
  // keeps the address space and emits shared-memory loads and stores instead of generic ones
  uint8_t* smem = smem_raw + ((1024u - (tw::smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* qFull = bars;
  uint64_t* kFull = qFull + 1;
  uint64_t* kEmpty = kFull + ATT_SLOTS;
  uint64_t* vFull = kEmpty + ATT_SLOTS;
  uint64_t* vEmpty = vFull + ATT_SLOTS;
  uint64_t* sFull = vEmpty + ATT_SLOTS;     // [2] scores of tile parity ready in TMEM
  uint64_t* sEmpty = sFull + 2;             // [2] softmax warps have read them
  uint64_t* pFull = sEmpty + 2;             // [2] P buffer written
  uint64_t* pEmpty = pFull + 2;             // [2] PV of that buffer finished
  uint64_t* tFull = pEmpty + 2;             // [1] (+1 spare) PV result ready in TMEM
  uint64_t* tEmpty = tFull + 2;
  uint64_t* statFull = tEmpty + 2;          // [4] (alpha, pf) of a key tile written
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(statFull + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* sel = smem + L::OFF_SEL;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int mb = blockIdx.x, h = blockIdx.y, kh = h / (p.hq / p.hk);
  const bool need_q1 = p.repair != 0;
  const bool need_k1 = p.repair && p.terms >= 3;
  const bool need_v1 = p.pv_repair && p.pv_terms >= 3;

  if (threadIdx.x == 0) {
    tw::mbar_init(qFull, 1);
    for (int i = 0; i < ATT_SLOTS; ++i) {
      tw::mbar_init(kFull + i, 1); tw::mbar_init(kEmpty + i, 4);   // the 4 softmax warps of the tile's group, after S and kf are consumed
      tw::mbar_init(vFull + i, 1); tw::mbar_init(vEmpty + i, 8);   // the 8 accumulate warps, after T and vf are consumed
    }
    for (int i = 0; i < 2; ++i) {
      tw::mbar_init(sFull + i, 1); tw::mbar_init(sEmpty + i, 4);
      tw::mbar_init(pFull + i, 4); tw::mbar_init(pEmpty + i, 1);
      tw::mbar_init(tFull + i, 1); tw::mbar_init(tEmpty + i, 8);
    }
    for (int i = 0; i < 4; ++i) tw::mbar_init(statFull + i, 4);
    *abort_flag = 0;
    tw::fence_barrier_init();
    tw::tma_prefetch_desc(&tm_q); tw::tma_prefetch_desc(&tm_k); tw::tma_prefetch_desc(&tm_v);
  }
  // per key tile: which repair terms are issued (read once; flags stay fixed during the launch)
  for (int t = threadIdx.x; t < p.nt; t += blockDim.x) {
    const size_t idx = ((size_t)h * p.mblk + mb) * p.nt + t;
    const bool qk = p.repair && (p.full || (p.flags && p.flags[idx] > 1));
    const bool pv = p.pv_repair && (p.pv_full || (p.pvflags && p.pvflags[idx] > 1));
    sel[t] = (uint8_t)((qk ? 1 : 0) | (pv ? 2 : 0));
  }
  if (warp == 1) { tw::tmem_alloc(tmem_slot, 512); tw::tmem_relinquish(); }
  tw::tc_fence_before();
  __syncthreads();
  tw::tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < 4) {
  tw::reg_budget_shrink<ATT_REGS_CONTROL>();
  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    // The whole warp walks the key tiles (warp-wide waits keep it converged); one elected lane issues the
    // copies of a tile: issued from a single-lane branch the same instructions cost tens of cycles each.
    {
      const int q_row = h * p.mp + mb * 128;
      if (tw::elect_one()) {
        tw::mbar_expect_tx(qFull, (need_q1 ? 2u : 1u) * (ATT_TILE + ATT_SF));
        tw::tma_load_2d(smem + L::OFF_Q, &tm_q, 0, q_row, qFull);
        tw::bulk_load(smem + L::OFF_SFQ, p.sfq + ((size_t)h * p.mblk + mb) * ATT_SF, ATT_SF, qFull);
        if (need_q1) {
          tw::tma_load_2d(smem + L::OFF_Q + ATT_TILE, &tm_q, 0, p.hq * p.mp + q_row, qFull);
          tw::bulk_load(smem + L::OFF_SFQ + ATT_SF, p.sfq + ((size_t)(p.hq + h) * p.mblk + mb) * ATT_SF, ATT_SF, qFull);
        }
      }
      __syncwarp();
      bool ok = true;
      for (int t = 0; t < p.nt && ok; ++t) {
        const uint32_t s = t % ATT_SLOTS, ph = (t / ATT_SLOTS) & 1;
        const bool k1 = need_k1 && (sel[t] & 1), v1 = need_v1 && (sel[t] & 2);
        ok = tw::mbar_wait_all(kEmpty + s, ph ^ 1, abort_flag);
        if (!ok) break;
        if (tw::elect_one()) {
          tw::mbar_expect_tx(kFull + s, (k1 ? 2u : 1u) * (ATT_TILE + ATT_SF) + 512u);
          tw::tma_load_2d(smem + L::OFF_K + s * 2 * ATT_TILE, &tm_k, 0, kh * p.np + t * 128, kFull + s);
          tw::bulk_load(smem + L::OFF_SFK + s * 2 * ATT_SF, p.sfk + ((size_t)kh * p.nt + t) * ATT_SF, ATT_SF, kFull + s);
          tw::bulk_load(smem + L::OFF_KF + s * 512, p.kf + (size_t)kh * p.np + t * 128, 512, kFull + s);
          if (k1) {
            tw::tma_load_2d(smem + L::OFF_K + (s * 2 + 1) * ATT_TILE, &tm_k, 0, (p.hk + kh) * p.np + t * 128, kFull + s);
            tw::bulk_load(smem + L::OFF_SFK + (s * 2 + 1) * ATT_SF, p.sfk + ((size_t)(p.hk + kh) * p.nt + t) * ATT_SF, ATT_SF, kFull + s);
          }
        }
        __syncwarp();
        ok = tw::mbar_wait_all(vEmpty + s, ph ^ 1, abort_flag);
        if (!ok) break;
        if (tw::elect_one()) {
          tw::mbar_expect_tx(vFull + s, (v1 ? 2u : 1u) * (ATT_TILE + ATT_SF) + 512u);
          tw::tma_load_2d(smem + L::OFF_V + s * 2 * ATT_TILE, &tm_v, 0, (kh * p.nt + t) * 128, vFull + s);
          tw::bulk_load(smem + L::OFF_SFV + s * 2 * ATT_SF, p.sfv + ((size_t)kh * p.nt + t) * ATT_SF, ATT_SF, vFull + s);
          tw::bulk_load(smem + L::OFF_VF + s * 512, p.vf + ((size_t)kh * p.nt + t) * 128, 512, vFull + s);
          if (v1) {
            tw::tma_load_2d(smem + L::OFF_V + (s * 2 + 1) * ATT_TILE, &tm_v, 0, ((p.hk + kh) * p.nt + t) * 128, vFull + s);
            tw::bulk_load(smem + L::OFF_SFV + (s * 2 + 1) * ATT_SF, p.sfv + ((size_t)(p.hk + kh) * p.nt + t) * ATT_SF, ATT_SF, vFull + s);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // Whole, converged warp; one elected lane issues the tcgen05 operations of a product (scale copies, MMAs,
    // commits) in one straight block.
    {
      constexpr uint32_t IDESC = tw::make_idesc_nvf4(128, 128);
      constexpr uint64_t D64 = (uint64_t(1) << 46) | (uint64_t(4) << 61) | (uint64_t(512 >> 4) << 32) | (uint64_t(1) << 16);
      constexpr uint64_t DSF = (uint64_t(1) << 46) | (uint64_t(128 >> 4) << 32);
      const uint32_t base = tw::smem_u32(smem);
      auto lo = [&](int off) { return (uint64_t)(((base + off) >> 4) & 0x3fffu); };
      auto copy_sf = [&](uint32_t tcol, int smem_off) {
        tw::tc_copy_scales(tmem + tcol, DSF | lo(smem_off));
        tw::tc_copy_scales(tmem + tcol + 4, DSF | lo(smem_off + 512));
      };
      auto mma = [&](uint32_t d, int a_off, int b_off, uint32_t sfa, uint32_t sfb, bool first) {
        tw::tc_mma_nvf4(tmem + d, D64 | lo(a_off), D64 | lo(b_off), IDESC, tmem + sfa, tmem + sfb, first ? 0u : 1u);
        tw::tc_mma_nvf4(tmem + d, D64 | lo(a_off + 32), D64 | lo(b_off + 32), IDESC, tmem + sfa + 4, tmem + sfb + 4, 1u);
      };
      bool ok = tw::mbar_wait_all(qFull, 0, abort_flag);
      tw::tc_fence_after();
      if (tw::elect_one()) {
        copy_sf(TM_SFQ0, L::OFF_SFQ);
        if (need_q1) copy_sf(TM_SFQ1, L::OFF_SFQ + ATT_SF);
      }
      __syncwarp();
      // scores of key tile t into S[t & 1]
      auto issue_qk = [&](int t) {
        const uint32_t s = t % ATT_SLOTS, ph = (t / ATT_SLOTS) & 1, par = t & 1;
        if (!tw::mbar_wait_all(kFull + s, ph, abort_flag) || !tw::mbar_wait_all(sEmpty + par, ((t >> 1) & 1) ^ 1, abort_flag)) return false;
        tw::tc_fence_after();
        const bool rep = sel[t] & 1;
        const int k0 = L::OFF_K + s * 2 * ATT_TILE, k1 = k0 + ATT_TILE;
        if (tw::elect_one()) {
          copy_sf(TM_SFK0 + par * 8, L::OFF_SFK + s * 2 * ATT_SF);
          mma(TM_S + par * 128, L::OFF_Q, k0, TM_SFQ0, TM_SFK0 + par * 8, true);
          if (rep) {
            mma(TM_S + par * 128, L::OFF_Q + ATT_TILE, k0, TM_SFQ1, TM_SFK0 + par * 8, false);
            if (p.terms >= 3) {
              copy_sf(TM_SFK1 + par * 8, L::OFF_SFK + (s * 2 + 1) * ATT_SF);
              mma(TM_S + par * 128, L::OFF_Q, k1, TM_SFQ0, TM_SFK1 + par * 8, false);
              if (p.terms == 4) mma(TM_S + par * 128, L::OFF_Q + ATT_TILE, k1, TM_SFQ1, TM_SFK1 + par * 8, false);
            }
          }
          tw::tc_commit(sFull + par);        // (the K slot is released by the softmax group once it has read kf)
        }
        __syncwarp();
        return true;
      };
      // S is double-buffered by tile parity = by softmax group. The scores of tile t + 2 are issued as soon as
      // the group of tile t has pulled S[t & 1] into registers (sEmpty), which is well before it posts P(t):
      // its next scores are ready when it comes back, instead of queueing behind the P V product.
      if (ok) ok = issue_qk(0);
      if (ok && p.nt > 1) ok = issue_qk(1);
      for (int t = 0; t < p.nt && ok; ++t) {
        if (t + 2 < p.nt) ok = issue_qk(t + 2);
        if (!ok) break;
        const uint32_t s = t % ATT_SLOTS, ph = (t / ATT_SLOTS) & 1, par = t & 1;
        const bool rep = sel[t] & 2;
        const int p0 = L::OFF_P + par * 2 * ATT_TILE, p1 = p0 + ATT_TILE;
        const int v0 = L::OFF_V + s * 2 * ATT_TILE, v1 = v0 + ATT_TILE;
        ok = tw::mbar_wait_all(vFull + s, ph, abort_flag) && tw::mbar_wait_all(pFull + par, (t >> 1) & 1, abort_flag) &&
             tw::mbar_wait_all(tEmpty, (t & 1) ^ 1, abort_flag);
        if (!ok) break;
        tw::tc_fence_after();
        if (tw::elect_one()) {
          copy_sf(TM_SFV0 + par * 8, L::OFF_SFV + s * 2 * ATT_SF);
          if (rep && p.pv_terms >= 3) copy_sf(TM_SFV1 + par * 8, L::OFF_SFV + (s * 2 + 1) * ATT_SF);
          copy_sf(TM_SFP0 + par * 8, L::OFF_SFP + par * 2 * ATT_SF);
          mma(TM_T, p0, v0, TM_SFP0 + par * 8, TM_SFV0 + par * 8, true);
          if (rep) {
            copy_sf(TM_SFP1 + par * 8, L::OFF_SFP + (par * 2 + 1) * ATT_SF);
            mma(TM_T, p1, v0, TM_SFP1 + par * 8, TM_SFV0 + par * 8, false);
            if (p.pv_terms >= 3) {
              mma(TM_T, p0, v1, TM_SFP0 + par * 8, TM_SFV1 + par * 8, false);
              if (p.pv_terms == 4) mma(TM_T, p1, v1, TM_SFP1 + par * 8, TM_SFV1 + par * 8, false);
            }
          }
          tw::tc_commit(tFull);              // (the V slot is released by the accumulate warps once they have read vf)
          tw::tc_commit(pEmpty + par);
        }
        __syncwarp();
      }
    }
  }
  } else if (warp < 12) {
    // ------------------------------------------------------------------ softmax and P quantization
    // Two groups of four warps; group g takes the key tiles of parity g (their scores live in S[g], their
    // probabilities in P[g]), so the two warps of every scheduler work on different tiles and the
    // conversion-unit-bound second pass of one runs beside the first pass and the waits of the other.
    // A thread owns one query row (TMEM lane) with all 128 key columns of the tile.
    // Everything runs in the log2 domain: x = S * kf[n] * (qf[m] * log2(e) / sqrt(128)). Each group keeps
    // its own lazy reference ref (raised only when a tile's row maximum exceeds it by more than 2^8);
    // the scaled probability z = p / pf is produced directly as exp2(x - off) with off = ref + log2(pf):
    // pf = max(exp2(rowmax - ref) / 1536, 1e-12) = exp2(off - ref),
    // off = max(rowmax - log2(1536), ref + log2(1e-12)).
    // (ref, pf, row sum) of each tile go to the accumulate warps through a ring of four slots.
    tw::reg_budget_grow<ATT_REGS_SOFTMAX>();
    const int quad = warp & 3, grp = (warp - 4) >> 2, r = quad * 32 + lane;
    const int m = mb * 128 + r;
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    const float qfl = (m < p.mp ? __ldg(p.qf + (size_t)h * p.mp + m) : 1.f) * (0.08838834764831845f * 1.4426950408889634f);
    float4* stats = reinterpret_cast<float4*>(smem + L::OFF_STAT);    // [4][128]: (ref, pf, row sum, -)
    float ref = -INFINITY;
    bool ok = true;
    // four code bytes (one per register, upper bits clear) -> one word, first byte lowest
    auto pack4 = [](uint32_t b0, uint32_t b1, uint32_t b2, uint32_t b3) {
      return __byte_perm(__byte_perm(b0, b1, 0x0040), __byte_perm(b2, b3, 0x0040), 0x5410);
    };
    // One key tile. TAIL: the tile holds padding columns (only the last tile of a ragged key length);
    // REP: the residual plane P1 is produced too. The loops over the four 32-column chunks stay rolled:
    // the body of a chunk is a few kilobytes of straight-line code and is reused from the instruction
    // cache, where the fully unrolled tile was refetched by every warp for every tile.
    float* gsm = reinterpret_cast<float*>(smem + L::OFF_GMAX) + grp * 8 * 128;   // [8 K16 groups][128 rows]
    auto tile = [&](int t, auto tail_tag, auto rep_tag) {
      constexpr bool TAIL = decltype(tail_tag)::value;
      constexpr bool REP = decltype(rep_tag)::value;
      const uint32_t s = t % ATT_SLOTS, ph = (t / ATT_SLOTS) & 1, par = grp;
      bool good = tw::mbar_wait(sFull + par, (t >> 1) & 1, abort_flag) && tw::mbar_wait(kFull + s, ph, abort_flag);
      good = __all_sync(0xffffffffu, good);
      if (!good) return false;
      tw::tc_fence_after();
      const float4* kf = reinterpret_cast<const float4*>(smem + L::OFF_KF + s * 512);
      const int n_valid = p.n - t * 128;                      // columns >= n_valid are padding
      // Both passes walk the 128 scores of the row in K16 groups with the tensor-memory load of the next group
      // in flight while the current one is processed (two 16-register buffers). The loads and their waits are
      // ordered among themselves and tied to the destination registers, but are no barrier for other
      // instructions: a thread runs long dependent chains (shared-memory load -> multiply -> exp2 -> convert ->
      // pack), and with two softmax warps per scheduler the only way to hide their latency is to let the
      // chains of neighbouring groups overlap. Arithmetic on pairs of columns uses the packed f32x2 forms,
      // which round exactly like two scalar operations.
      const uint32_t s_src = lane_base + TM_S + par * 128;
      auto walk = [&](auto&& process, auto&& last_load_done) {
        uint32_t va[16], vb[16];
        tw::tmem_load_16_async(s_src, va);
        tw::tmem_load_wait(va);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          tw::tmem_load_16_async(s_src + c * 32 + 16, vb);
          process(va, c, std::integral_constant<int, 0>{});
          tw::tmem_load_wait(vb);
          if (c < 3) tw::tmem_load_16_async(s_src + c * 32 + 32, va);
          else last_load_done();
          process(vb, c, std::integral_constant<int, 1>{});
          if (c < 3) tw::tmem_load_wait(va);
        }
      };
      // products S * kf of columns 4 i .. 4 i + 3 of a K16 group, as two pairs
      auto scaled = [&](const uint32_t (&v)[16], int c, int g, int i, float2& e0, float2& e1) {
        const float4 f = kf[c * 8 + g * 4 + i];
        e0 = __fmul2_rn(make_float2(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1])), make_float2(f.x, f.y));
        e1 = __fmul2_rn(make_float2(__uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3])), make_float2(f.z, f.w));
      };
      // pass 1: maximum of S * kf per K16 group
      float rowmax = -INFINITY;
      walk([&](const uint32_t (&v)[16], int c, auto g_tag) {
        constexpr int g = decltype(g_tag)::value;
        float part[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 e0, e1;
          scaled(v, c, g, i, e0, e1);
          if (TAIL) {
            const int col = c * 32 + g * 16 + 4 * i;
            if (col >= n_valid) e0.x = -INFINITY;
            if (col + 1 >= n_valid) e0.y = -INFINITY;
            if (col + 2 >= n_valid) e1.x = -INFINITY;
            if (col + 3 >= n_valid) e1.y = -INFINITY;
          }
          part[i] = fmaxf(fmaxf(e0.x, e0.y), fmaxf(e1.x, e1.y));
        }
        const float best = fmaxf(fmaxf(part[0], part[1]), fmaxf(part[2], part[3]));
        gsm[(c * 2 + g) * 128 + r] = best;
        rowmax = fmaxf(rowmax, best);
      }, [] {});
      rowmax *= qfl;                                          // qfl > 0
      if (rowmax > ref + 8.f) ref = rowmax;                   // lazy reference
      const float off = fmaxf(rowmax - 10.584962500721156f, ref - 39.863137138648348f);
      const float pf = exp2_approx(off - ref);
      // the P buffer of this parity must have been consumed by the PV product two tiles ago
      good = tw::mbar_wait(pEmpty + par, ((t >> 1) & 1) ^ 1, abort_flag);
      good = __all_sync(0xffffffffu, good);
      if (!good) return false;
      uint8_t* p0 = smem + L::OFF_P + par * 2 * ATT_TILE;
      uint8_t* sfp = smem + L::OFF_SFP + par * 2 * ATT_SF;
      float zsum = 0.f;
      uint32_t sf_base = 0u, sf_res = 0u;
      uint32_t w[4], rw[4];
      const float2 q2 = make_float2(qfl, qfl);
      // pass 2: per K16 group the E4M3 scale follows from the group maximum, and the codes are the E2M1
      // roundings of y = exp2(x - off - log2(scale)) = z / scale
      // scale of a K16 group from its maximum: E4M3 byte, its value, and the exponent offset of the group. The
      // chain (exp2 -> convert -> convert back -> log2) is long, so the one of the next group is started before
      // the columns of the current group are processed.
      float next_sv, next_offg;
      uint32_t next_sb;
      auto group_scale = [&](int group) {
        const float peak = exp2_approx(__fmaf_rn(gsm[group * 128 + r], qfl, -off));
        next_sb = tw::f32_to_e4m3(fmaxf(peak * (1.f / 6.f), 0.001953125f));
        next_sv = tw::e4m3_to_f32(next_sb);
        next_offg = off + lg2_approx(next_sv);
      };
      group_scale(0);
      walk([&](const uint32_t (&v)[16], int c, auto g_tag) {
        constexpr int g = decltype(g_tag)::value;
        const uint32_t sb = next_sb;
        const float sv = next_sv, offg = next_offg;
        if (g == 0 || c < 3) group_scale(c * 2 + g + 1);
        const float2 o2 = make_float2(-offg, -offg);
        float2 y[8];
        float2 ysum = make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 e0, e1;
          scaled(v, c, g, i, e0, e1);
          e0 = __ffma2_rn(e0, q2, o2);
          e1 = __ffma2_rn(e1, q2, o2);
          y[2 * i] = make_float2(exp2_approx(e0.x), exp2_approx(e0.y));
          y[2 * i + 1] = make_float2(exp2_approx(e1.x), exp2_approx(e1.y));
          if (TAIL) {
            const int col = c * 32 + g * 16 + 4 * i;
            if (col >= n_valid) y[2 * i].x = 0.f;
            if (col + 1 >= n_valid) y[2 * i].y = 0.f;
            if (col + 2 >= n_valid) y[2 * i + 1].x = 0.f;
            if (col + 3 >= n_valid) y[2 * i + 1].y = 0.f;
          }
          ysum = __fadd2_rn(ysum, __fadd2_rn(y[2 * i], y[2 * i + 1]));
        }
        zsum = __fmaf_rn(ysum.x + ysum.y, sv, zsum);
        uint32_t b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = tw::f32x2_to_e2m1x2(y[i].x, y[i].y);
        w[2 * g] = pack4(b[0], b[1], b[2], b[3]);
        w[2 * g + 1] = pack4(b[4], b[5], b[6], b[7]);
        sf_base |= sb << (8 * ((c & 1) * 2 + g));
        if (REP) {
          // residual in units of the base scale: res = y - value(code); its scale is sv * max|res| / 6
          float rpeak = 0.f;
          const float2 minus = make_float2(-1.f, -1.f);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            y[i] = __ffma2_rn(e2m1x2_values(b[i]), minus, y[i]);
            rpeak = fmaxf(rpeak, fmaxf(fabsf(y[i].x), fabsf(y[i].y)));
          }
          const uint32_t rsb = tw::f32_to_e4m3(fmaxf(rpeak * sv * (1.f / 6.f), 0.001953125f));
          const float mult = sv * rcp_approx(tw::e4m3_to_f32(rsb));
          const float2 m2 = make_float2(mult, mult);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float2 scaled_res = __fmul2_rn(y[i], m2);
            b[i] = tw::f32x2_to_e2m1x2(scaled_res.x, scaled_res.y);
          }
          rw[2 * g] = pack4(b[0], b[1], b[2], b[3]);
          rw[2 * g + 1] = pack4(b[4], b[5], b[6], b[7]);
          sf_res |= rsb << (8 * ((c & 1) * 2 + g));
        }
        if (g == 1) {
          // K16 groups 2c and 2c + 1 of a row share one 16-byte chunk of the 64-byte-swizzled P tile
          const uint32_t code_off = (uint32_t)r * 64u + (uint32_t)((c ^ ((r >> 1) & 3)) << 4);
          *reinterpret_cast<uint4*>(p0 + code_off) = make_uint4(w[0], w[1], w[2], w[3]);
          if (REP) *reinterpret_cast<uint4*>(p0 + ATT_TILE + code_off) = make_uint4(rw[0], rw[1], rw[2], rw[3]);
          if (c & 1) {                                        // four scale bytes of the row: one word of the atom layout
            *reinterpret_cast<uint32_t*>(sfp + atom_offset(r, (c >> 1) * 4)) = sf_base;
            if (REP) *reinterpret_cast<uint32_t*>(sfp + ATT_SF + atom_offset(r, (c >> 1) * 4)) = sf_res;
            sf_base = sf_res = 0u;
          }
        }
      }, [&] {                                                // all scores are in registers: release S[par]
        tw::tc_fence_before();
        __syncwarp();
        if (lane == 0) tw::mbar_arrive(sEmpty + par);
      });
      stats[(t & 3) * 128 + r] = make_float4(ref, pf, zsum * pf, 0.f);
      // P visible to the tensor core (async proxy); key factors consumed
      tw::fence_proxy_async();
      __syncwarp();
      if (lane == 0) { tw::mbar_arrive(kEmpty + s); tw::mbar_arrive(pFull + par); tw::mbar_arrive(statFull + (t & 3)); }
      return true;
    };
    const bool ragged = (p.n & 127) != 0;
    for (int t = grp; t < p.nt && ok; t += 2) {
      const bool rep = sel[t] & 2;
      if (ragged && t == p.nt - 1) ok = rep ? tile(t, std::true_type{}, std::true_type{}) : tile(t, std::true_type{}, std::false_type{});
      else ok = rep ? tile(t, std::false_type{}, std::true_type{}) : tile(t, std::false_type{}, std::false_type{});
    }
  } else {
    // ------------------------------------------------------------------ accumulate and output
    // Eight warps, two per TMEM lane quadrant: a thread owns one query row and 64 of the 128 channels.
    // Per key tile, with (ref, pf, sum) of the row from the softmax group that handled it:
    //   R' = ref if ref > R + 2^8 else R;  alpha = 2^(R - R');  w = 2^(ref - R')
    //   acc = acc * alpha + T * (pf * w) * vf;   den = den * alpha + sum * w
    // fp32, in registers; the rescaling multiply is skipped when alpha is 1 for the whole warp.
    tw::reg_budget_grow<ATT_REGS_ACCUM>();
    const int quad = warp & 3, half = (warp - 12) >> 2, r = quad * 32 + lane;
    const int m = mb * 128 + r, c0 = half * 64;
    const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
    const float4* stats = reinterpret_cast<const float4*>(smem + L::OFF_STAT);
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    float R = -INFINITY, den = 0.f;
    bool ok = true;
    for (int t = 0; t < p.nt && ok; ++t) {
      const uint32_t s = t % ATT_SLOTS, ph = (t / ATT_SLOTS) & 1;
      ok = tw::mbar_wait(statFull + (t & 3), (t >> 2) & 1, abort_flag) && tw::mbar_wait(tFull, t & 1, abort_flag) &&
           tw::mbar_wait(vFull + s, ph, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const float4 st = stats[(t & 3) * 128 + r];
      const float Rn = st.x > R + 8.f ? st.x : R;
      const float alpha = exp2_approx(R - Rn), wgt = exp2_approx(st.x - Rn);
      const float pf = st.y * wgt;
      den = __fmaf_rn(den, alpha, st.z * wgt);
      R = Rn;
      const bool keep = __all_sync(0xffffffffu, alpha == 1.f);
      tw::tc_fence_after();
      const float4* vf = reinterpret_cast<const float4*>(smem + L::OFF_VF + s * 512) + (c0 >> 2);
      // T is read 16 columns at a time with the next load in flight; the T buffer is handed back to the MMA warp
      // as soon as the last load has landed, before the last columns are accumulated. Pairs of channels use the
      // packed f32x2 forms (same rounding as two scalar operations).
      const float2 pf2 = make_float2(pf, pf), alpha2 = make_float2(alpha, alpha);
      auto accumulate = [&](const uint32_t (&v)[16], int c) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 f = vf[c * 4 + i];
          float2* a0 = reinterpret_cast<float2*>(&acc[c * 16 + 4 * i]);
          float2* a1 = reinterpret_cast<float2*>(&acc[c * 16 + 4 * i + 2]);
          const float2 t0 = __fmul2_rn(make_float2(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1])), make_float2(f.x, f.y));
          const float2 t1 = __fmul2_rn(make_float2(__uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3])), make_float2(f.z, f.w));
          if (keep) {
            *a0 = __ffma2_rn(t0, pf2, *a0);
            *a1 = __ffma2_rn(t1, pf2, *a1);
          } else {
            *a0 = __ffma2_rn(t0, pf2, __fmul2_rn(*a0, alpha2));
            *a1 = __ffma2_rn(t1, pf2, __fmul2_rn(*a1, alpha2));
          }
        }
      };
      {
        uint32_t va[16], vb[16];
        const uint32_t t_src = lane_base + TM_T + c0;
        tw::tmem_load_16_async(t_src, va);
        tw::tmem_load_wait(va);
        tw::tmem_load_16_async(t_src + 16, vb);
        accumulate(va, 0);
        tw::tmem_load_wait(vb);
        tw::tmem_load_16_async(t_src + 32, va);
        accumulate(vb, 1);
        tw::tmem_load_wait(va);
        tw::tmem_load_16_async(t_src + 48, vb);
        accumulate(va, 2);
        tw::tmem_load_wait(vb);
        tw::tc_fence_before();
        __syncwarp();
        if (lane == 0) tw::mbar_arrive(tEmpty);
        accumulate(vb, 3);
      }
      __syncwarp();
      if (lane == 0) tw::mbar_arrive(vEmpty + s);
    }
    if (ok && m < p.m) {
      const float inv = 1.f / den;
      __nv_bfloat16* dst = p.out + ((size_t)m * p.hq + h) * 128 + c0;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          __nv_bfloat162 b2 = __floats2bfloat162_rn(acc[16 * j + 2 * q] * inv, acc[16 * j + 2 * q + 1] * inv);
          w[q] = *reinterpret_cast<uint32_t*>(&b2);
        }
        tw::store_256(dst + 16 * j, w);
      }
    }
  }

  tw::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TW_ERR_TIMEOUT);
  if (warp == 1) { tw::tc_fence_after(); tw::tmem_dealloc(tmem, 512); }
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// C entry points
// ---------------------------------------------------------------------------------------------
namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn att_encode_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      f = nullptr;
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}
// [rows, 64 bytes] code matrix, boxes of 128 rows, 64-byte swizzle
bool code_map(CUtensorMap* map, const void* base, size_t rows) {
  cuuint64_t dims[2] = {64, (cuuint64_t)rows};
  cuuint64_t strides[1] = {64};
  cuuint32_t box[2] = {64, 128}, ones[2] = {1, 1};
  return att_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, ones,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace

extern "C" int tw_pack_rows(const TwPackRowsArgs* a, void* stream_) {
  if (!a || !a->x || !a->codes || !a->scales || !a->scales_swz || !a->factors) return TW_ERR_ARGUMENT;
  if (a->rows <= 0 || a->heads <= 0 || a->rows_padded < a->rows) return TW_ERR_ARGUMENT;
  if (a->transpose_v ? (a->rows_padded % 128 != 0) : (a->rows_padded % 16 != 0)) return TW_ERR_SHAPE;
  if (a->need_energy && (!a->transpose_v || !a->energy)) return TW_ERR_ARGUMENT;
  if (((uintptr_t)a->x | (uintptr_t)a->codes | (uintptr_t)a->scales | (uintptr_t)a->scales_swz) & 15) return TW_ERR_ALIGNMENT;
  if ((a->stride_row | a->stride_head) & 7) return TW_ERR_ALIGNMENT;      // 16-byte vector loads
  RowPackParams p{};
  p.x = static_cast<const __nv_bfloat16*>(a->x);
  p.codes = a->codes; p.scales = a->scales; p.scales_swz = a->scales_swz; p.factors = a->factors; p.energy = a->energy;
  p.stride_row = a->stride_row; p.stride_head = a->stride_head;
  p.rows = a->rows; p.heads = a->heads; p.rows_padded = a->rows_padded; p.blocks128 = (a->rows_padded + 127) / 128;
  p.repair = a->repair; p.need_energy = a->need_energy;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a->transpose_v) pack_v_kernel<<<dim3(a->rows_padded / 128, a->heads), 256, 0, stream>>>(p);
  else pack_qk_kernel<<<dim3((a->rows_padded + 31) / 32, a->heads), 256, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

extern "C" int tw_select_tiles(const TwSelectArgs* a, void* stream_) {
  if (!a || !a->q || !a->k || !a->energy || !a->flags || !a->counts) return TW_ERR_ARGUMENT;
  if (a->m <= 0 || a->n <= 0 || a->hq <= 0 || a->hk <= 0 || a->hq % a->hk) return TW_ERR_ARGUMENT;
  if (a->pvflags && !a->pvcounts) return TW_ERR_ARGUMENT;
  if ((((uintptr_t)a->q | (uintptr_t)a->k) & 15) || ((a->q_stride_row | a->q_stride_head | a->k_stride_row | a->k_stride_head) & 7))
    return TW_ERR_ALIGNMENT;                                // 16-byte row loads
  SelectParams p{};
  p.q = static_cast<const __nv_bfloat16*>(a->q); p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.energy = a->energy; p.flags = a->flags; p.pvflags = a->pvflags; p.counts = a->counts; p.pvcounts = a->pvcounts;
  p.q_row = a->q_stride_row; p.q_head = a->q_stride_head; p.k_row = a->k_stride_row; p.k_head = a->k_stride_head;
  p.m = a->m; p.n = a->n; p.hq = a->hq; p.hk = a->hk; p.nt = (a->n + 127) / 128; p.terms = a->terms; p.pvterms = a->pv_terms;
  const size_t smem = (8 * 128 + 8 * p.nt * 8 + p.nt) * sizeof(float);
  if (smem > 200 * 1024) return TW_ERR_TOO_LARGE;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return TW_ERR_LAUNCH;
  select_kernel<<<dim3(a->hq, (a->m + 127) / 128), 128, smem, static_cast<cudaStream_t>(stream_)>>>(p);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

extern "C" size_t tw_attention_workspace(int, int, int, int) { return 256; }

extern "C" int tw_attention(const TwAttentionArgs* a, void* stream_) {
  if (!a || !a->qc || !a->kc || !a->vc || !a->sfq || !a->sfk || !a->sfv || !a->qf || !a->kf || !a->vf || !a->out ||
      !a->workspace)
    return TW_ERR_ARGUMENT;
  if (a->m <= 0 || a->n <= 0 || a->hq <= 0 || a->hk <= 0 || a->hq % a->hk) return TW_ERR_ARGUMENT;
  if (a->mp != (a->m + 15) / 16 * 16 || a->np != (a->n + 127) / 128 * 128) return TW_ERR_SHAPE;
  if (a->terms < 2 || a->terms > 4 || a->pv_terms < 2 || a->pv_terms > 4) return TW_ERR_ARGUMENT;
  const int nt = a->np / 128, mblk = (a->mp + 127) / 128;
  if (nt > ATT_NT_MAX) return TW_ERR_TOO_LARGE;
  if (a->repair && !a->full && !a->flags) return TW_ERR_ARGUMENT;
  if (a->pv_repair && !a->pv_full && !a->pvflags) return TW_ERR_ARGUMENT;
  // TMA bases and bulk copies need 16-byte alignment; the output rows are written with 32-byte stores
  const uintptr_t align16 = (uintptr_t)a->qc | (uintptr_t)a->kc | (uintptr_t)a->vc | (uintptr_t)a->sfq | (uintptr_t)a->sfk |
                            (uintptr_t)a->sfv | (uintptr_t)a->qf | (uintptr_t)a->kf | (uintptr_t)a->vf;
  if ((align16 & 15) || ((uintptr_t)a->out & 31)) return TW_ERR_ALIGNMENT;
  if (!att_encode_fn()) return TW_ERR_DRIVER;
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TW_ERR_LAUNCH;
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (major != 10) return TW_ERR_ARCH;
  const int q_planes = a->repair ? 2 : 1;
  const int k_planes = (a->repair && a->terms >= 3) ? 2 : 1;
  const int v_planes = (a->pv_repair && a->pv_terms >= 3) ? 2 : 1;
  CUtensorMap tm_q, tm_k, tm_v;
  if (!code_map(&tm_q, a->qc, (size_t)q_planes * a->hq * a->mp) || !code_map(&tm_k, a->kc, (size_t)k_planes * a->hk * a->np) ||
      !code_map(&tm_v, a->vc, (size_t)v_planes * a->hk * a->np))
    return TW_ERR_TENSOR_MAP;
  AttParams p{};
  p.sfq = a->sfq; p.sfk = a->sfk; p.sfv = a->sfv; p.qf = a->qf; p.kf = a->kf; p.vf = a->vf;
  p.flags = a->flags; p.pvflags = a->pvflags;
  p.out = static_cast<__nv_bfloat16*>(a->out); p.status = static_cast<int*>(a->workspace);
  p.m = a->m; p.n = a->n; p.hq = a->hq; p.hk = a->hk; p.mp = a->mp; p.np = a->np; p.mblk = mblk; p.nt = nt;
  p.repair = a->repair; p.full = a->full; p.terms = a->terms;
  p.pv_repair = a->pv_repair; p.pv_full = a->pv_full; p.pv_terms = a->pv_terms;
  // the shared-memory opt-in is a per-device attribute of the function
  static std::atomic<bool> configured[64];
  if (!configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttSmem::BYTES) != cudaSuccess)
      return TW_ERR_LAUNCH;
    // the in-kernel register rebalance assumes the launch allocation it was sized for
    cudaFuncAttributes attr;
    if (cudaFuncGetAttributes(&attr, attention_kernel) != cudaSuccess || attr.numRegs < ATT_REGS_LAUNCH) return TW_ERR_LAUNCH;
    configured[dev].store(true, std::memory_order_release);
  }
  attention_kernel<<<dim3((a->m + 127) / 128, a->hq), ATT_THREADS, AttSmem::BYTES, static_cast<cudaStream_t>(stream_)>>>(tm_q, tm_k, tm_v, p);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}
