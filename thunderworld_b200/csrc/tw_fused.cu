// Fused selective-repair GEMM for sm_100a.
//
//   out = alpha * ( A0 W0^T + A1 W0^T|a-support + A0 W1^T|w-tiles [+ A1 W1^T|both] )      bf16 [M,N]
//
// All operands are NVFP4 (E2M1 codes, one UE4M3 scale per 16 k). Every term is issued as
// tcgen05.mma kind::mxf4nvf4.block_scale into ONE fp32 accumulator in tensor memory; the epilogue
// scales by the device scalar alpha and rounds to bf16 once. Term structure follows the reference
// (thunderworld_fp4/_native.py:11-62; cutlass/repair_collective.cuh:117-132); what differs is the
// schedule: terms are interleaved per K128 block so that each operand tile is fetched once per
// output tile: per kb the CTA loads A0[kb], W0[kb], A1[kb] if selected and the W1 tiles of (nb,kb),
// and issues A0W0, A1W0, A0W1, A1W1 back to back.
//
// CTA = one 128 x BN output tile at a time (persistent over tiles), warp-specialised:
//   warp 0      producer: TMA loads of code tiles (64-byte swizzle) + bulk copies of scale atoms
//   warp 1      MMA issuer: scale atoms smem -> TMEM (tcgen05.cp), MMAs, commits
//   warp 2      builds the per-tile term tables (A-support bytes, W1 bank positions) ahead of use
//   warps 4-11  epilogue: TMEM -> registers -> bf16 -> global (16-byte stores), TMEM released first
// Operand rings: A slots (128 rows x 64 B codes + 1 KB scales), W0 slots (BN rows x 64 B codes +
// BN/128 KB scales) and W1 slots (128 rows). No cluster, no multicast.
#include <cuda.h>
#include "tw_common.cuh"
#include "../../include/twb200.h"

namespace {

constexpr int KB_MAX = 256;               // K <= 32768
constexpr int A_TILE = 128 * 64;          // bytes of one 128 x K128 code tile
constexpr int SF_ATOM = 1024;             // bytes of the scales of 128 rows x K128

template <int BN> struct Cfg {
  static constexpr int HALVES = BN / 128;
  static constexpr int A_SLOTS = 7;                           // A0 / A1 tiles
  static constexpr int B_SLOTS = BN == 256 ? 6 : 8;           // W0 tiles (BN rows)
  static constexpr int W_SLOTS = 4;                           // W1 tiles (128 rows)
  static constexpr int TAB_SLOTS = 3;                         // per-tile term tables built ahead
  static constexpr int ACC_STAGES = BN == 256 ? 1 : 2;
  static constexpr int EPI_WARPS = 8;
  static constexpr int FIRST_EPI_WARP = 4;                    // warps 0..3: producer, MMA, tables, spare
  static constexpr int EPI_GROUPS = EPI_WARPS / 4;            // column groups per lane quadrant
  static constexpr int EPI_COLS = BN / EPI_GROUPS;            // columns per epilogue warp
  static constexpr int THREADS = (FIRST_EPI_WARP + EPI_WARPS) * 32;
  static constexpr int B_TILE = BN * 64;
  // shared-memory carve-up (offsets from a 1024-aligned base)
  static constexpr int OFF_A = 0;
  static constexpr int OFF_B = OFF_A + A_SLOTS * A_TILE;
  static constexpr int OFF_W = OFF_B + B_SLOTS * B_TILE;
  static constexpr int OFF_SFA = OFF_W + W_SLOTS * A_TILE;
  static constexpr int OFF_SFB = OFF_SFA + A_SLOTS * SF_ATOM;
  static constexpr int OFF_SFW = OFF_SFB + B_SLOTS * HALVES * SF_ATOM;
  static constexpr int OFF_TAB = OFF_SFW + W_SLOTS * SF_ATOM;
  static constexpr int TAB_BYTES = HALVES * KB_MAX * 4 + KB_MAX;
  static constexpr int OFF_BAR = OFF_TAB + TAB_SLOTS * TAB_BYTES;
  static constexpr int NUM_BARS = 2 * A_SLOTS + 2 * B_SLOTS + 2 * W_SLOTS + 2 * TAB_SLOTS + 2 * ACC_STAGES;
  static constexpr int SMEM_BYTES = OFF_BAR + NUM_BARS * 8 + 64 + 1024;  // + alignment slack
  // tensor-memory columns
  static constexpr int TM_ACC = 0;
  static constexpr int TM_SF = ACC_STAGES * BN;                          // 256
  static constexpr int TM_SFA0 = TM_SF, TM_SFA1 = TM_SF + 16, TM_SFB0 = TM_SF + 32, TM_SFBW = TM_SF + 32 + 2 * 4 * HALVES * 2;
  static constexpr int TM_COLS = 512;
};
static_assert(Cfg<256>::SMEM_BYTES <= 232448 && Cfg<128>::SMEM_BYTES <= 232448, "shared memory budget");

struct Params {
  const uint8_t* sfa0;      // atom-layout scales of A0  [MB*128, K/16]
  const uint8_t* sfa1;      // atom-layout scales of A1
  const uint8_t* sfb0;      // atom-layout scales of W0  [N, K/16]
  const uint8_t* sfbw;      // atom-layout scales of the W1 bank, 1 KB per tile
  const int* wi; const int* off; const int* wloc;
  const uint8_t* mask;
  const float* alpha;
  __nv_bfloat16* out;
  int* status;
  int m, mp, n, k, na, hasw, cross, shared, dense;
  int kb, nb, mb, tiles_n, tiles;
};

// Per-tile term table: for every kb whether A1 is selected and, for each N128 half of the tile,
// the bank position of the W1 tile at (nb, kb) or -1.
template <int BN> struct TermTable {
  int w1[Cfg<BN>::HALVES][KB_MAX];
  uint8_t a1[KB_MAX];
};

template <int BN>
__device__ __forceinline__ void build_table(TermTable<BN>& tab, const Params& p, int mbi, int nt, int lane) {
  constexpr int H = Cfg<BN>::HALVES;
  int begin[H], end[H];
#pragma unroll
  for (int h = 0; h < H; ++h) {
    const int nb = nt * H + h;
    const bool use = p.hasw && !p.dense && nb < p.nb;
    begin[h] = use ? p.off[nb] : 0;
    end[h] = use ? p.off[nb + 1] : 0;
  }
  for (int kb = lane; kb < p.kb; kb += 32) {
    tab.a1[kb] = p.na == p.kb ? 1 : (p.na > 0 ? p.mask[mbi * p.kb + kb] : 0);
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const int nb = nt * H + h;
      tab.w1[h][kb] = (p.hasw && p.dense && nb < p.nb) ? nb * p.kb + kb : -1;
    }
  }
  __syncwarp();
#pragma unroll
  for (int h = 0; h < H; ++h)
    for (int s = begin[h] + lane; s < end[h]; s += 32) tab.w1[h][p.wi[s]] = p.shared ? p.wloc[s] : s;
  __syncwarp();
}

template <int BN>
__global__ void __launch_bounds__(Cfg<BN>::THREADS, 1)
fused_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w0,
             const __grid_constant__ CUtensorMap tm_w1, const Params p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem + C::OFF_A;
  uint8_t* sB = smem + C::OFF_B;
  uint8_t* sW = smem + C::OFF_W;
  uint8_t* sSFA = smem + C::OFF_SFA;
  uint8_t* sSFB = smem + C::OFF_SFB;
  uint8_t* sSFW = smem + C::OFF_SFW;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* fullA = bars;
  uint64_t* emptyA = fullA + C::A_SLOTS;
  uint64_t* fullB = emptyA + C::A_SLOTS;
  uint64_t* emptyB = fullB + C::B_SLOTS;
  uint64_t* fullW = emptyB + C::B_SLOTS;
  uint64_t* emptyW = fullW + C::W_SLOTS;
  uint64_t* tabFull = emptyW + C::W_SLOTS;
  uint64_t* tabEmpty = tabFull + C::TAB_SLOTS;
  uint64_t* accFull = tabEmpty + C::TAB_SLOTS;
  uint64_t* accEmpty = accFull + C::ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accEmpty + C::ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto table = [&](uint32_t i) -> TermTable<BN>& {
    return *reinterpret_cast<TermTable<BN>*>(smem + C::OFF_TAB + (i % C::TAB_SLOTS) * C::TAB_BYTES);
  };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::A_SLOTS; ++i) { tw::mbar_init(fullA + i, 1); tw::mbar_init(emptyA + i, 1); }
    for (int i = 0; i < C::B_SLOTS; ++i) { tw::mbar_init(fullB + i, 1); tw::mbar_init(emptyB + i, 1); }
    for (int i = 0; i < C::W_SLOTS; ++i) { tw::mbar_init(fullW + i, 1); tw::mbar_init(emptyW + i, 1); }
    for (int i = 0; i < C::TAB_SLOTS; ++i) { tw::mbar_init(tabFull + i, 1); tw::mbar_init(tabEmpty + i, 2); }
    for (int i = 0; i < C::ACC_STAGES; ++i) { tw::mbar_init(accFull + i, 1); tw::mbar_init(accEmpty + i, C::EPI_WARPS); }
    *abort_flag = 0;
    tw::fence_barrier_init();
    tw::tma_prefetch_desc(&tm_a); tw::tma_prefetch_desc(&tm_w0); tw::tma_prefetch_desc(&tm_w1);
  }
  if (warp == 1) { tw::tmem_alloc(tmem_slot, C::TM_COLS); tw::tmem_relinquish(); }
  tw::tc_fence_before();
  __syncthreads();
  tw::tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 2) {
    // ------------------------------------------------------------------ term tables, built ahead
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
      ok = tw::mbar_wait(tabEmpty + it % C::TAB_SLOTS, ((it / C::TAB_SLOTS) & 1) ^ 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      build_table<BN>(table(it), p, tile / p.tiles_n, tile % p.tiles_n, lane);
      if (lane == 0) tw::mbar_arrive(tabFull + it % C::TAB_SLOTS);
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ producer (one thread)
    if (lane == 0) {
      uint32_t ia = 0, ib = 0, iw = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
        const int mbi = tile / p.tiles_n, nt = tile % p.tiles_n;
        const TermTable<BN>& tab = table(it);
        ok = tw::mbar_wait(tabFull + it % C::TAB_SLOTS, (it / C::TAB_SLOTS) & 1, abort_flag);
        const int n_rows = min(BN, p.n - nt * BN);            // 128 or BN
        for (int kb = 0; kb < p.kb && ok; ++kb) {
          const bool sel = tab.a1[kb] != 0;
          auto load_a = [&](int plane) {
            const uint32_t s = ia % C::A_SLOTS, ph = (ia / C::A_SLOTS) & 1; ++ia;
            if (!tw::mbar_wait(emptyA + s, ph ^ 1, abort_flag)) return false;
            tw::mbar_expect_tx(fullA + s, A_TILE + SF_ATOM);
            tw::tma_load_3d(sA + s * A_TILE, &tm_a, kb * 64, mbi * 128, plane, fullA + s);
            const uint8_t* sf = (plane ? p.sfa1 : p.sfa0) + ((size_t)mbi * p.kb + kb) * SF_ATOM;
            tw::bulk_load(sSFA + s * SF_ATOM, sf, SF_ATOM, fullA + s);
            return true;
          };
          ok = load_a(0);
          if (!ok) break;
          {
            const uint32_t s = ib % C::B_SLOTS, ph = (ib / C::B_SLOTS) & 1; ++ib;
            ok = tw::mbar_wait(emptyB + s, ph ^ 1, abort_flag);
            if (!ok) break;
            tw::mbar_expect_tx(fullB + s, (uint32_t)n_rows * 64 + (uint32_t)(n_rows / 128) * SF_ATOM);
            tw::tma_load_2d(sB + s * C::B_TILE, &tm_w0, kb * 64, nt * BN, fullB + s);
            for (int h = 0; h < n_rows / 128; ++h) {
              const uint8_t* sf = p.sfb0 + ((size_t)(nt * C::HALVES + h) * p.kb + kb) * SF_ATOM;
              tw::bulk_load(sSFB + (s * C::HALVES + h) * SF_ATOM, sf, SF_ATOM, fullB + s);
            }
          }
          if (sel) { ok = load_a(1); if (!ok) break; }
          for (int h = 0; h < C::HALVES && ok; ++h) {
            const int loc = tab.w1[h][kb];
            if (loc < 0) continue;
            const uint32_t s = iw % C::W_SLOTS, ph = (iw / C::W_SLOTS) & 1; ++iw;
            ok = tw::mbar_wait(emptyW + s, ph ^ 1, abort_flag);
            if (!ok) break;
            tw::mbar_expect_tx(fullW + s, A_TILE + SF_ATOM);
            tw::tma_load_2d(sW + s * A_TILE, &tm_w1, 0, loc * 128, fullW + s);
            tw::bulk_load(sSFW + s * SF_ATOM, p.sfbw + (size_t)loc * SF_ATOM, SF_ATOM, fullW + s);
          }
        }
        tw::mbar_arrive(tabEmpty + it % C::TAB_SLOTS);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    if (lane == 0) {
      uint32_t ia = 0, ib = 0, iw = 0, it = 0;
      bool ok = true;
      constexpr uint32_t IDESC_FULL = tw::make_idesc_nvf4(128, BN);
      constexpr uint32_t IDESC_128 = tw::make_idesc_nvf4(128, 128);
      const uint64_t desc_hi = tw::make_smem_desc(0, 16, 512, 4);   // 64-byte swizzle, 8-row groups 512 B apart
      const uint64_t sf_hi = tw::make_smem_desc(0, 0, 128, 0);      // scale atom: 32 rows x 16 B, no swizzle
      auto op_desc = [&](uint32_t addr) { return desc_hi | (uint64_t)((addr >> 4) & 0x3fffu); };
      auto sf_desc = [&](uint32_t addr) { return sf_hi | (uint64_t)((addr >> 4) & 0x3fffu); };
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
        const int nt = tile % p.tiles_n;
        const TermTable<BN>& tab = table(it);
        ok = tw::mbar_wait(tabFull + it % C::TAB_SLOTS, (it / C::TAB_SLOTS) & 1, abort_flag);
        const int n_rows = min(BN, p.n - nt * BN);
        const uint32_t idesc_base = n_rows == BN ? IDESC_FULL : IDESC_128;
        const uint32_t stage = it % C::ACC_STAGES, aph = (it / C::ACC_STAGES) & 1;
        ok = ok && tw::mbar_wait(accEmpty + stage, aph ^ 1, abort_flag);
        tw::tc_fence_after();
        const uint32_t acc = tmem + C::TM_ACC + stage * BN;
        for (int kb = 0; kb < p.kb && ok; ++kb) {
          const bool sel = tab.a1[kb] != 0;
          const uint32_t par = kb & 1;                           // double-buffered TMEM scale regions
          const uint32_t t_sfa0 = tmem + C::TM_SFA0 + par * 8, t_sfa1 = tmem + C::TM_SFA1 + par * 8;
          const uint32_t t_sfb0 = tmem + C::TM_SFB0 + par * 8 * C::HALVES;
          // A0 and W0
          const uint32_t sa0 = ia % C::A_SLOTS, pa0 = (ia / C::A_SLOTS) & 1; ++ia;
          const uint32_t sb0 = ib % C::B_SLOTS, pb0 = (ib / C::B_SLOTS) & 1; ++ib;
          ok = tw::mbar_wait(fullA + sa0, pa0, abort_flag) && tw::mbar_wait(fullB + sb0, pb0, abort_flag);
          if (!ok) break;
          tw::tc_fence_after();
          const uint32_t a0_addr = tw::smem_u32(sA + sa0 * A_TILE), b0_addr = tw::smem_u32(sB + sb0 * C::B_TILE);
          const uint32_t sfa0_addr = tw::smem_u32(sSFA + sa0 * SF_ATOM), sfb0_addr = tw::smem_u32(sSFB + sb0 * C::HALVES * SF_ATOM);
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            tw::tc_copy_scales(t_sfa0 + 4 * c, sf_desc(sfa0_addr + c * 512));
#pragma unroll
            for (int h = 0; h < C::HALVES; ++h)
              if (h * 128 < n_rows)
                tw::tc_copy_scales(t_sfb0 + 4 * C::HALVES * c + 4 * h, sf_desc(sfb0_addr + h * SF_ATOM + c * 512));
          }
#pragma unroll
          for (int c = 0; c < 2; ++c)
            tw::tc_mma_nvf4(acc, op_desc(a0_addr + 32 * c), op_desc(b0_addr + 32 * c), idesc_base, t_sfa0 + 4 * c,
                            t_sfb0 + 4 * C::HALVES * c, (kb | c) != 0);
          // A1 against the same W0 tile
          uint32_t sa1 = 0, a1_addr = 0;
          if (sel) {
            sa1 = ia % C::A_SLOTS; const uint32_t pa1 = (ia / C::A_SLOTS) & 1; ++ia;
            ok = tw::mbar_wait(fullA + sa1, pa1, abort_flag);
            if (!ok) break;
            tw::tc_fence_after();
            a1_addr = tw::smem_u32(sA + sa1 * A_TILE);
            const uint32_t sfa1_addr = tw::smem_u32(sSFA + sa1 * SF_ATOM);
#pragma unroll
            for (int c = 0; c < 2; ++c) tw::tc_copy_scales(t_sfa1 + 4 * c, sf_desc(sfa1_addr + c * 512));
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tw::tc_mma_nvf4(acc, op_desc(a1_addr + 32 * c), op_desc(b0_addr + 32 * c), idesc_base, t_sfa1 + 4 * c,
                              t_sfb0 + 4 * C::HALVES * c, 1u);
          }
          tw::tc_commit(emptyB + sb0);
          // W1 tiles of this kb: 128-column MMAs into the matching half of the accumulator
          for (int h = 0; h < C::HALVES && ok; ++h) {
            if (tab.w1[h][kb] < 0) continue;
            const uint32_t sw = iw % C::W_SLOTS, pw = (iw / C::W_SLOTS) & 1;
            const uint32_t t_sfbw = tmem + C::TM_SFBW + ((iw & 1) * 8);
            ++iw;
            ok = tw::mbar_wait(fullW + sw, pw, abort_flag);
            if (!ok) break;
            tw::tc_fence_after();
            const uint32_t bw_addr = tw::smem_u32(sW + sw * A_TILE), sfw_addr = tw::smem_u32(sSFW + sw * SF_ATOM);
#pragma unroll
            for (int c = 0; c < 2; ++c) tw::tc_copy_scales(t_sfbw + 4 * c, sf_desc(sfw_addr + c * 512));
#pragma unroll
            for (int c = 0; c < 2; ++c)
              tw::tc_mma_nvf4(acc + h * 128, op_desc(a0_addr + 32 * c), op_desc(bw_addr + 32 * c), IDESC_128,
                              t_sfa0 + 4 * c, t_sfbw + 4 * c, 1u);
            if (p.cross && sel) {
#pragma unroll
              for (int c = 0; c < 2; ++c)
                tw::tc_mma_nvf4(acc + h * 128, op_desc(a1_addr + 32 * c), op_desc(bw_addr + 32 * c), IDESC_128,
                                t_sfa1 + 4 * c, t_sfbw + 4 * c, 1u);
            }
            tw::tc_commit(emptyW + sw);
          }
          tw::tc_commit(emptyA + sa0);
          if (sel) tw::tc_commit(emptyA + sa1);
        }
        if (ok) tw::tc_commit(accFull + stage);
        tw::mbar_arrive(tabEmpty + it % C::TAB_SLOTS);
      }
    }
  } else if (warp >= C::FIRST_EPI_WARP) {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;                              // TMEM lane quadrant this warp may read
    const int group = (warp - C::FIRST_EPI_WARP) >> 2;      // column group
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
      const int mbi = tile / p.tiles_n, nt = tile % p.tiles_n;
      const uint32_t stage = it % C::ACC_STAGES, aph = (it / C::ACC_STAGES) & 1;
      ok = tw::mbar_wait(accFull + stage, aph, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tw::tc_fence_after();
      const float alpha = __ldg(p.alpha);
      const uint32_t t_base = tmem + ((uint32_t)(quad * 32) << 16) + C::TM_ACC + stage * BN + group * C::EPI_COLS;
      uint32_t packed[C::EPI_COLS / 2];
#pragma unroll
      for (int part = 0; part < C::EPI_COLS / 32; ++part) {
        uint32_t r[32];
        tw::tmem_load_32x32(t_base + part * 32, r);
        tw::tmem_load_wait();
#pragma unroll
        for (int q = 0; q < 16; ++q) {
          __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(r[2 * q]) * alpha, __uint_as_float(r[2 * q + 1]) * alpha);
          packed[part * 16 + q] = *reinterpret_cast<uint32_t*>(&b);
        }
      }
      // accumulator drained into registers: hand the TMEM stage back before storing
      tw::tc_fence_before();
      __syncwarp();
      if (lane == 0) tw::mbar_arrive(accEmpty + stage);
      const int row = mbi * 128 + quad * 32 + lane;
      const int col = nt * BN + group * C::EPI_COLS;
      if (row < p.m && col < p.n) {
        uint4* dst = reinterpret_cast<uint4*>(p.out + (size_t)row * p.n + col);
#pragma unroll
        for (int j = 0; j < C::EPI_COLS / 8; ++j)
          dst[j] = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
      }
    }
  }

  tw::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TW_ERR_TIMEOUT);
  if (warp == 1) { tw::tc_fence_after(); tw::tmem_dealloc(tmem, C::TM_COLS); }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

bool make_map(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const cuuint64_t* dims,
              const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swz) {
  cuuint32_t ones[3] = {1, 1, 1};
  return encode_fn()(map, type, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, ones,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN>
int launch(int m, int n, int k, const void* a_codes, const void* w_codes, const void* sfa, const void* sfb, void* out,
           const float* alpha, void* workspace, cudaStream_t stream, const TwRepairIO* io, int sms) {
  using C = Cfg<BN>;
  CUtensorMap tm_a, tm_w0, tm_w1;
  const int planes = io->na > 0 ? 2 : 1;
  {
    cuuint64_t dims[3] = {(cuuint64_t)k / 2, (cuuint64_t)io->mp, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)k / 2, (cuuint64_t)io->mp * (k / 2)};
    cuuint32_t box[3] = {64, 128, 1};
    if (!make_map(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a_codes, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B))
      return TW_ERR_TENSOR_MAP;
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)k / 2, (cuuint64_t)n};
    cuuint64_t strides[1] = {(cuuint64_t)k / 2};
    cuuint32_t box[2] = {64, (cuuint32_t)(n >= BN ? BN : 128)};
    if (!make_map(&tm_w0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w_codes, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B))
      return TW_ERR_TENSOR_MAP;
  }
  {
    const bool has = io->hasw != 0;
    cuuint64_t dims[2] = {64, (cuuint64_t)(has ? (size_t)io->bank_blocks * 128 : 128)};
    cuuint64_t strides[1] = {64};
    cuuint32_t box[2] = {64, 128};
    if (!make_map(&tm_w1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, has ? (const void*)io->wr : w_codes, dims, strides, box,
                  CU_TENSOR_MAP_SWIZZLE_64B))
      return TW_ERR_TENSOR_MAP;
  }
  Params p{};
  p.sfa0 = static_cast<const uint8_t*>(sfa);
  p.sfa1 = io->a1s_swz;
  p.sfb0 = static_cast<const uint8_t*>(sfb);
  p.sfbw = io->wrs_swz;
  p.wi = io->wi; p.off = io->off; p.wloc = io->wloc; p.mask = io->mask;
  p.alpha = alpha;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = static_cast<int*>(workspace);
  p.m = m; p.mp = io->mp; p.n = n; p.k = k; p.na = io->na; p.hasw = io->hasw; p.cross = io->cross;
  p.shared = io->shared; p.dense = io->dense;
  p.kb = k / 128; p.nb = n / 128; p.mb = (m + 127) / 128;
  p.tiles_n = (n + BN - 1) / BN;
  p.tiles = p.mb * p.tiles_n;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(fused_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
      return TW_ERR_LAUNCH;
    configured = true;
  }
  const int grid = p.tiles < sms ? p.tiles : sms;
  fused_kernel<BN><<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(tm_a, tm_w0, tm_w1, p);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

}  // namespace

extern "C" size_t tw_workspace(int, int, int) { return 256; }

extern "C" int tw_fused_tile_n(int n) { return n % 256 == 0 ? 256 : 128; }

extern "C" int tw_fused(int m, int n, int k, const void* a_codes, const void* w_codes, const void* sfa, const void* sfb,
                        void* out, const float* alpha, void* workspace, void* stream, const TwRepairIO* io) {
  if (!io || !a_codes || !w_codes || !sfa || !sfb || !out || !alpha || !workspace) return TW_ERR_ARGUMENT;
  if (m <= 0 || n <= 0 || k <= 0) return TW_ERR_ARGUMENT;
  if (n % 128 || k % 128 || k / 128 > KB_MAX) return TW_ERR_SHAPE;
  if (io->m != m || io->n != n || io->k != k || io->mp != (m + 15) / 16 * 16) return TW_ERR_SHAPE;
  if (io->na < 0 || io->na > k / 128) return TW_ERR_ARGUMENT;
  if (io->na > 0 && !io->a1s_swz) return TW_ERR_MISSING_SWIZZLED;
  if (io->na > 0 && io->na < k / 128 && !io->mask) return TW_ERR_ARGUMENT;
  if (io->hasw) {
    if (!io->wr || !io->wrs_swz) return TW_ERR_MISSING_SWIZZLED;
    if (io->bank_blocks <= 0) return TW_ERR_ARGUMENT;
    if (!io->dense && (!io->wi || !io->off)) return TW_ERR_ARGUMENT;
    if (io->shared && !io->wloc) return TW_ERR_ARGUMENT;
  }
  const uintptr_t align = (uintptr_t)a_codes | (uintptr_t)w_codes | (uintptr_t)sfa | (uintptr_t)sfb | (uintptr_t)out |
                          (uintptr_t)io->a1s_swz | (uintptr_t)io->wrs_swz | (uintptr_t)io->wr;
  if (align & 15) return TW_ERR_ALIGNMENT;
  if (!encode_fn()) return TW_ERR_DRIVER;
  int dev = 0, sms = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return TW_ERR_LAUNCH;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (major != 10) return TW_ERR_ARCH;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n % 256 == 0) return launch<256>(m, n, k, a_codes, w_codes, sfa, sfb, out, alpha, workspace, s, io, sms);
  return launch<128>(m, n, k, a_codes, w_codes, sfa, sfb, out, alpha, workspace, s, io, sms);
}
