// Fused selective-repair GEMM for sm_100a.
//
//   out = alpha * ( A0 W0^T + A1 W0^T|a-support + A0 W1^T|w-tiles [+ A1 W1^T|both] )      bf16 [M,N]
//
// All operands are NVFP4 (E2M1 codes, one UE4M3 scale per 16 k). Every term is issued as
// tcgen05.mma kind::mxf4nvf4.block_scale into ONE fp32 accumulator in tensor memory; the epilogue
// scales by the device scalar alpha and rounds to bf16 once. Term structure follows the reference
// (thunderworld_fp4/_native.py:11-62; cutlass/repair_collective.cuh:117-132); what differs is the
// schedule. The K loop advances in steps of 256 (two blocks of the K128 repair lattice): a "base
// stage" holds A0 (128 x 128 B) and W0 (BN x 128 B) of the step with their scales and costs the
// single-thread producer and MMA roles one barrier round trip; the repair operands of the same
// step (A1 blocks, W1 tiles: "units" of 128 x 64 B) arrive through a second ring and are multiplied
// against the resident base stage, so W0 is fetched once for A0 and A1, and A0 once for W0 and W1.
//
// CTA = one 128 x BN output tile at a time (persistent over tiles), warp-specialised:
//   warp 0      producer of base stages (TMA, 128-byte swizzle; bulk copies of scale atoms)
//   warp 1      MMA issuer: MMAs, scale copies of repair units, commits
//   warps 2, 6  producers of repair units (A1 blocks / W1 tiles; TMA, 64-byte swizzle)
//   warp 3      builds the per-tile term tables (A-support bits, W1 bank positions) ahead of use
//   warps 4,5   copy the base-stage scale atoms smem -> TMEM (tcgen05.cp) ahead of the MMA issuer
//   warps 8-15  epilogue: TMEM -> registers -> bf16 -> global (32-byte stores)
// No cluster, no multicast.
#include <atomic>
#include <cuda.h>
#include "tw_common.cuh"
#include "../../include/twb200.h"

namespace {

constexpr int KB_MAX = 192;               // K <= 24576
constexpr int UNIT_TILE = 128 * 64;       // bytes of one 128-row x K128 code tile
constexpr int SF_ATOM = 1024;             // bytes of the scales of 128 rows x K128

// DEEP = true trades one base stage for deeper repair-unit rings: at the 2x plan a K256 step takes long
// enough for two base stages, and the issuer waits less for unit scales; without repair terms the third
// base stage is worth 16 %. The host picks the variant from the plan.
template <int BN, bool DEEP = false> struct Cfg {
  static constexpr int HALVES = BN / 128;
  static constexpr int STAGES = BN == 256 ? (DEEP ? 2 : 3) : 4;   // base stages (K256 of A0 and W0)
  static constexpr int A1_SLOTS = DEEP && BN == 256 ? 4 : 3;      // A1 units
  static constexpr int W1_SLOTS = DEEP && BN == 256 ? 6 : 3;      // W1 units
  static constexpr int TAB_SLOTS = 3;                         // per-tile term tables built ahead
  static constexpr int ACC_STAGES = BN == 256 ? 1 : 2;
  static constexpr int EPI_WARPS = 8;
  static constexpr int FIRST_EPI_WARP = 8;                    // warps 0-3 and 4-5 are single-thread roles, 6-7 idle
  static constexpr int SF_THREADS = 2;                        // threads that copy base-stage scales into TMEM
  static constexpr int EPI_GROUPS = EPI_WARPS / 4;            // column groups per lane quadrant
  static constexpr int EPI_COLS = BN / EPI_GROUPS;            // columns per epilogue warp
  static constexpr int THREADS = (FIRST_EPI_WARP + EPI_WARPS) * 32;
  static constexpr int A0_TILE = 128 * 128;                   // 128 rows x K256
  static constexpr int W0_TILE = BN * 128;
  static constexpr int STAGE_SF = (1 + HALVES) * 2 * SF_ATOM; // A0 scales then W0 scales per half
  // shared-memory carve-up (offsets from a 1024-aligned base)
  static constexpr int OFF_A0 = 0;
  static constexpr int OFF_W0 = OFF_A0 + STAGES * A0_TILE;
  static constexpr int OFF_A1 = OFF_W0 + STAGES * W0_TILE;
  static constexpr int OFF_W1 = OFF_A1 + A1_SLOTS * UNIT_TILE;
  static constexpr int OFF_SF0 = OFF_W1 + W1_SLOTS * UNIT_TILE;
  static constexpr int OFF_SFA1 = OFF_SF0 + STAGES * STAGE_SF;
  static constexpr int OFF_SFW1 = OFF_SFA1 + A1_SLOTS * SF_ATOM;
  static constexpr int OFF_TAB = OFF_SFW1 + W1_SLOTS * SF_ATOM;
  static constexpr int TAB_BYTES = HALVES * KB_MAX * 4 + (HALVES + 1) * (KB_MAX / 32) * 4;
  static constexpr int OFF_BAR = OFF_TAB + TAB_SLOTS * TAB_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 2 * A1_SLOTS + 2 * W1_SLOTS + 2 * TAB_SLOTS + 2 * ACC_STAGES + STAGES + A1_SLOTS + W1_SLOTS;
  static constexpr int SMEM_BYTES = OFF_BAR + NUM_BARS * 8 + 64 + 1024;  // + alignment slack
  // tensor-memory columns: accumulators, then double-buffered scale regions
  static constexpr int TM_ACC = 0;
  static constexpr int TM_SFA0 = ACC_STAGES * BN;                        // STAGES x 16 columns: one region per smem stage
  static constexpr int TM_SFB0 = TM_SFA0 + 16 * STAGES;                  // STAGES x 16*HALVES columns
  static constexpr int TM_SFA1 = TM_SFB0 + 16 * HALVES * STAGES;                  // 8 columns per A1 slot
  static constexpr int TM_SFW1 = TM_SFA1 + 32;                           // 8 columns per W1 slot
  static constexpr int TM_COLS = 512;
  static_assert(A1_SLOTS * 8 <= 32 && TM_SFW1 + 8 * W1_SLOTS <= TM_COLS, "tensor memory budget");
};
static_assert(Cfg<256>::SMEM_BYTES <= 232448 && Cfg<256, true>::SMEM_BYTES <= 232448 && Cfg<128>::SMEM_BYTES <= 232448,
              "shared memory budget");

struct Params {
  const uint8_t* sfa0;      // atom-layout scales of A0  [MB*128, K/16]
  const uint8_t* sfa1;      // atom-layout scales of A1
  const uint8_t* sfb0;      // atom-layout scales of W0  [N, K/16]
  const uint8_t* sfbw;      // atom-layout scales of the W1 bank, 1 KB per tile
  const int* wi; const int* off; const int* wloc;
  const uint8_t* mask;
  const float* alpha;
  const __nv_bfloat16* bias;  // optional [n], added in fp32 before the bf16 rounding
  __nv_bfloat16* out;
  int* status;
  int m, mp, n, k, na, hasw, cross, shared, dense;
  int kb, nb, mb, tiles_n, tiles;
  int mask_per_n;           // mask is [MB, NB, KB] (one A support per output block; 128-wide tiles only)
};

// Per-tile term table, built ahead of use by its own warp: one bit per kb for "A1 selected" and
// for "a W1 tile exists at (nb, kb)" per N128 half of the tile (the MMA issuer and the producers
// walk these bits in registers), and the bank position of each W1 tile for the unit producer.
template <int BN> struct TermTable {
  int w1loc[Cfg<BN>::HALVES][KB_MAX];
  uint32_t w1bits[Cfg<BN>::HALVES][KB_MAX / 32];
  uint32_t a1bits[KB_MAX / 32];
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
  const int words = (p.kb + 31) / 32;
  for (int w = 0; w < words; ++w) {
    const int kb = w * 32 + lane;
    const bool in = kb < p.kb;
    const size_t mrow = p.mask_per_n ? (size_t)mbi * p.nb + nt : (size_t)mbi;
    const bool sel = in && ((p.na == p.kb && !p.mask_per_n) || (p.na > 0 && p.mask[mrow * p.kb + kb] != 0));
    const uint32_t abits = __ballot_sync(0xffffffffu, sel);
    if (lane == 0) tab.a1bits[w] = abits;
#pragma unroll
    for (int h = 0; h < H; ++h) {
      const bool dense = in && p.hasw && p.dense && (nt * H + h) < p.nb;
      if (in) tab.w1loc[h][kb] = dense ? (nt * H + h) * p.kb + kb : -1;
      const uint32_t wb = __ballot_sync(0xffffffffu, dense);
      if (lane == 0) tab.w1bits[h][w] = wb;
    }
  }
  __syncwarp();
#pragma unroll
  for (int h = 0; h < H; ++h)
    for (int s = begin[h] + lane; s < end[h]; s += 32) {
      const int kb = p.wi[s];
      tab.w1loc[h][kb] = p.shared ? p.wloc[s] : s;
      atomicOr(&tab.w1bits[h][kb >> 5], 1u << (kb & 31));
    }
  __syncwarp();
}

template <int BN, bool DEEP>
__global__ void __launch_bounds__(Cfg<BN, DEEP>::THREADS, 1)
fused_kernel(const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_a1,
             const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1, const Params p) {
  using C = Cfg<BN, DEEP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* fullS = bars;                       // base stages
  uint64_t* emptyS = fullS + C::STAGES;
  uint64_t* fullA1 = emptyS + C::STAGES;        // A1 units
  uint64_t* emptyA1 = fullA1 + C::A1_SLOTS;
  uint64_t* fullW1 = emptyA1 + C::A1_SLOTS;     // W1 units
  uint64_t* emptyW1 = fullW1 + C::W1_SLOTS;
  uint64_t* tabFull = emptyW1 + C::W1_SLOTS;
  uint64_t* tabEmpty = tabFull + C::TAB_SLOTS;
  uint64_t* accFull = tabEmpty + C::TAB_SLOTS;
  uint64_t* accEmpty = accFull + C::ACC_STAGES;
  uint64_t* sfFull = accEmpty + C::ACC_STAGES;   // scales of the base stage in slot i are in its TMEM region
  uint64_t* usfA = sfFull + C::STAGES;                  // scales of the A1 unit in slot i are in TMEM
  uint64_t* usfW = usfA + C::A1_SLOTS;           // same for W1 units
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(usfW + C::W1_SLOTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto table = [&](uint32_t i) -> TermTable<BN>& {
    return *reinterpret_cast<TermTable<BN>*>(smem + C::OFF_TAB + (i % C::TAB_SLOTS) * C::TAB_BYTES);
  };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int steps = (p.kb + 1) / 2;             // K256 steps; the last one may hold a single K128 block

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::STAGES; ++i) { tw::mbar_init(fullS + i, 1); tw::mbar_init(emptyS + i, 1); }
    for (int i = 0; i < C::A1_SLOTS; ++i) { tw::mbar_init(fullA1 + i, 1); tw::mbar_init(emptyA1 + i, 1); }
    for (int i = 0; i < C::W1_SLOTS; ++i) { tw::mbar_init(fullW1 + i, 1); tw::mbar_init(emptyW1 + i, 1); }
    for (int i = 0; i < C::TAB_SLOTS; ++i) { tw::mbar_init(tabFull + i, 1); tw::mbar_init(tabEmpty + i, 3 + C::SF_THREADS); }
    for (int i = 0; i < C::ACC_STAGES; ++i) { tw::mbar_init(accFull + i, 1); tw::mbar_init(accEmpty + i, C::EPI_WARPS); }
    for (int i = 0; i < C::STAGES; ++i) tw::mbar_init(sfFull + i, C::SF_THREADS);
    for (int i = 0; i < C::A1_SLOTS; ++i) tw::mbar_init(usfA + i, 1);
    for (int i = 0; i < C::W1_SLOTS; ++i) tw::mbar_init(usfW + i, 1);
    *abort_flag = 0;
    tw::fence_barrier_init();
    tw::tma_prefetch_desc(&tm_a0); tw::tma_prefetch_desc(&tm_a1);
    tw::tma_prefetch_desc(&tm_w0); tw::tma_prefetch_desc(&tm_w1);
  }
  if (warp == 1) { tw::tmem_alloc(tmem_slot, C::TM_COLS); tw::tmem_relinquish(); }
  tw::tc_fence_before();
  __syncthreads();
  tw::tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 3) {
    // ------------------------------------------------------------------ term tables, built ahead
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++it) {
      if (!tw::mbar_wait_warp(tabEmpty + it % C::TAB_SLOTS, ((it / C::TAB_SLOTS) & 1) ^ 1, abort_flag)) break;
      build_table<BN>(table(it), p, tile / p.tiles_n, tile % p.tiles_n, lane);
      if (lane == 0) tw::mbar_arrive(tabFull + it % C::TAB_SLOTS);
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ producer of base stages
    // Needs no term table: one stage per K256 step of every tile.
    if (lane == 0) {
      uint32_t is = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x) {
        const int mbi = tile / p.tiles_n, nt = tile % p.tiles_n;
        const int n_rows = min(BN, p.n - nt * BN);            // 128 or BN
        for (int st = 0; st < steps && ok; ++st, ++is) {
          const uint32_t s = is % C::STAGES, ph = (is / C::STAGES) & 1;
          const int kb0 = 2 * st, nk = min(2, p.kb - kb0);     // K128 blocks in this step
          ok = tw::mbar_wait(emptyS + s, ph ^ 1, abort_flag);
          if (!ok) break;
          // TMA always delivers the full box (out-of-range K reads as zero codes)
          tw::mbar_expect_tx(fullS + s, C::A0_TILE + (uint32_t)n_rows * 128 + (uint32_t)(1 + n_rows / 128) * nk * SF_ATOM);
          tw::tma_load_3d(smem + C::OFF_A0 + s * C::A0_TILE, &tm_a0, kb0 * 64, mbi * 128, 0, fullS + s);
          tw::tma_load_2d(smem + C::OFF_W0 + s * C::W0_TILE, &tm_w0, kb0 * 64, nt * BN, fullS + s);
          uint8_t* sf = smem + C::OFF_SF0 + s * C::STAGE_SF;
          tw::bulk_load(sf, p.sfa0 + ((size_t)mbi * p.kb + kb0) * SF_ATOM, nk * SF_ATOM, fullS + s);
          for (int h = 0; h < n_rows / 128; ++h)
            tw::bulk_load(sf + (1 + h) * 2 * SF_ATOM, p.sfb0 + ((size_t)(nt * C::HALVES + h) * p.kb + kb0) * SF_ATOM,
                          nk * SF_ATOM, fullS + s);
        }
      }
    }
  } else if (warp == 2 || warp == 6) {
    // ------------------------------------------------------------------ producers of repair units
    // Per step, in the order the MMA issuer consumes them: A1(kb0), A1(kb1) by warp 2, W1 tiles by
    // (kb, half) by warp 6: a full W1 ring does not hold the A1 loads of the next step back.
    if (lane == 0) {
      const bool do_a = warp == 2, do_w = warp == 6;
      uint32_t ia = 0, iw = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
        const int mbi = tile / p.tiles_n;
        const TermTable<BN>& tab = table(it);
        ok = tw::mbar_wait(tabFull + it % C::TAB_SLOTS, (it / C::TAB_SLOTS) & 1, abort_flag);
        uint32_t abits = 0, wbits[C::HALVES] = {};
        for (int st = 0; st < steps && ok; ++st) {
          const int kb0 = 2 * st;
          if ((kb0 & 31) == 0) {
            abits = tab.a1bits[kb0 >> 5];
#pragma unroll
            for (int h = 0; h < C::HALVES; ++h) wbits[h] = tab.w1bits[h][kb0 >> 5];
          }
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            if (!do_a || !((abits >> j) & 1u) || !ok) continue;
            const uint32_t s = ia % C::A1_SLOTS, ph = (ia / C::A1_SLOTS) & 1; ++ia;
            ok = tw::mbar_wait(emptyA1 + s, ph ^ 1, abort_flag);
            if (!ok) continue;
            tw::mbar_expect_tx(fullA1 + s, UNIT_TILE + SF_ATOM);
            tw::tma_load_3d(smem + C::OFF_A1 + s * UNIT_TILE, &tm_a1, (kb0 + j) * 64, mbi * 128, 1, fullA1 + s);
            tw::bulk_load(smem + C::OFF_SFA1 + s * SF_ATOM, p.sfa1 + ((size_t)mbi * p.kb + kb0 + j) * SF_ATOM, SF_ATOM, fullA1 + s);
          }
#pragma unroll
          for (int j = 0; j < 2; ++j) {
#pragma unroll
            for (int h = 0; h < C::HALVES; ++h) {
              if (!do_w || !((wbits[h] >> j) & 1u) || !ok) continue;
              const int loc = tab.w1loc[h][kb0 + j];
              const uint32_t s = iw % C::W1_SLOTS, ph = (iw / C::W1_SLOTS) & 1; ++iw;
              ok = tw::mbar_wait(emptyW1 + s, ph ^ 1, abort_flag);
              if (!ok) continue;
              tw::mbar_expect_tx(fullW1 + s, UNIT_TILE + SF_ATOM);
              tw::tma_load_2d(smem + C::OFF_W1 + s * UNIT_TILE, &tm_w1, 0, loc * 128, fullW1 + s);
              tw::bulk_load(smem + C::OFF_SFW1 + s * SF_ATOM, p.sfbw + (size_t)loc * SF_ATOM, SF_ATOM, fullW1 + s);
            }
          }
          abits >>= 2;
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) wbits[h] >>= 2;
        }
        tw::mbar_arrive(tabEmpty + it % C::TAB_SLOTS);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one thread)
    // One thread issues every tcgen05 operation, so its instruction stream is kept short: slot
    // counters advance incrementally, descriptors are a constant high word plus (address >> 4).
    if (lane == 0) {
      bool ok = true;
      constexpr uint32_t IDESC_FULL = tw::make_idesc_nvf4(128, BN);
      constexpr uint32_t IDESC_128 = tw::make_idesc_nvf4(128, 128);
      constexpr uint64_t D128 = (uint64_t(1) << 46) | (uint64_t(2) << 61) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 16);
      constexpr uint64_t D64 = (uint64_t(1) << 46) | (uint64_t(4) << 61) | (uint64_t(512 >> 4) << 32) | (uint64_t(1) << 16);
      constexpr uint64_t DSF = (uint64_t(1) << 46) | (uint64_t(128 >> 4) << 32);
      const uint32_t smem_u = tw::smem_u32(smem);
      const uint32_t a0_base = (smem_u + C::OFF_A0) >> 4, w0_base = (smem_u + C::OFF_W0) >> 4;
      const uint32_t a1_base = (smem_u + C::OFF_A1) >> 4, w1_base = (smem_u + C::OFF_W1) >> 4;
      const uint32_t t_sfa0_b = tmem + C::TM_SFA0, t_sfb0_b = tmem + C::TM_SFB0;
      uint32_t s = 0, ph = 0;                  // base stage slot / phase
      uint32_t sa = 0, pa = 0, sw = 0, pw = 0; // unit slots / phases
      uint32_t it = 0, tsl = 0, tph = 0;       // tile counter, table slot / phase
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
        const int nt = tile % p.tiles_n;
        const TermTable<BN>& tab = *reinterpret_cast<const TermTable<BN>*>(smem + C::OFF_TAB + tsl * C::TAB_BYTES);
        const int n_rows = min(BN, p.n - nt * BN);
        const uint32_t idesc_base = n_rows == BN ? IDESC_FULL : IDESC_128;
        const uint32_t stage = it % C::ACC_STAGES, aph = (it / C::ACC_STAGES) & 1;
        ok = tw::mbar_wait(tabFull + tsl, tph, abort_flag) && tw::mbar_wait(accEmpty + stage, aph ^ 1, abort_flag);
        tw::tc_fence_after();
        const uint32_t acc = tmem + C::TM_ACC + stage * BN;
        uint32_t abits = 0, wbits[C::HALVES] = {};
        for (int st = 0; st < steps && ok; ++st) {
          const int kb0 = 2 * st;
          const int nq = p.kb - kb0 >= 2 ? 4 : 2;                  // K64 slices in this step
          if ((kb0 & 31) == 0) {
            abits = tab.a1bits[kb0 >> 5];
#pragma unroll
            for (int h = 0; h < C::HALVES; ++h) wbits[h] = tab.w1bits[h][kb0 >> 5];
          }
          // the scale-copy threads waited for the stage's data and moved its scales into TMEM
          ok = tw::mbar_wait(sfFull + s, ph, abort_flag) && tw::mbar_wait(fullS + s, ph, abort_flag);
          if (!ok) break;
          tw::tc_fence_after();
          const uint32_t a0_lo = a0_base + s * (C::A0_TILE >> 4), w0_lo = w0_base + s * (C::W0_TILE >> 4);
          const uint32_t t_sfa0 = t_sfa0_b + s * 16, t_sfb0 = t_sfb0_b + s * 16 * C::HALVES;
#pragma unroll
          for (int q = 0; q < 4; ++q)                              // A0 W0
            if (q < nq)
              tw::tc_mma_nvf4(acc, D128 | (a0_lo + 2 * q), D128 | (w0_lo + 2 * q), idesc_base, t_sfa0 + 4 * q,
                              t_sfb0 + 4 * C::HALVES * q, (st | q) != 0);
          const uint32_t ab = abits & 3u;
          uint32_t wb = 0;
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) wb |= (wbits[h] & 3u) << (2 * h);
          if (ab | wb) {
            // A1 blocks of this step against the resident W0 stage
            uint32_t a1_lo[2] = {0, 0}, a1_bar[2] = {0, 0};
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              if (!((ab >> j) & 1u) || !ok) continue;
              ok = tw::mbar_wait(usfA + sa, pa, abort_flag);       // data landed and its scales are in TMEM
              if (!ok) continue;
              tw::tc_fence_after();
              a1_lo[j] = a1_base + sa * (UNIT_TILE >> 4);
              a1_bar[j] = sa;
              const uint32_t t_sfa1 = tmem + C::TM_SFA1 + sa * 8;
#pragma unroll
              for (int c = 0; c < 2; ++c)
                tw::tc_mma_nvf4(acc, D64 | (a1_lo[j] + 2 * c), D128 | (w0_lo + 4 * j + 2 * c), idesc_base,
                                t_sfa1 + 4 * c, t_sfb0 + 4 * C::HALVES * (2 * j + c), 1u);
              if (!p.cross) tw::tc_commit(emptyA1 + sa);
              if (++sa == C::A1_SLOTS) { sa = 0; pa ^= 1; }
            }
            // W1 tiles of this step: 128-column MMAs into the matching half of the accumulator
#pragma unroll
            for (int j = 0; j < 2; ++j) {
#pragma unroll
              for (int h = 0; h < C::HALVES; ++h) {
                if (!((wb >> (2 * h + j)) & 1u) || !ok) continue;
                ok = tw::mbar_wait(usfW + sw, pw, abort_flag);
                if (!ok) continue;
                tw::tc_fence_after();
                const uint32_t w1_lo = w1_base + sw * (UNIT_TILE >> 4);
                const uint32_t t_sfw1 = tmem + C::TM_SFW1 + sw * 8;
#pragma unroll
                for (int c = 0; c < 2; ++c)
                  tw::tc_mma_nvf4(acc + h * 128, D128 | (a0_lo + 4 * j + 2 * c), D64 | (w1_lo + 2 * c), IDESC_128,
                                  t_sfa0 + 4 * (2 * j + c), t_sfw1 + 4 * c, 1u);
                if (p.cross && ((ab >> j) & 1u)) {
                  const uint32_t t_sfa1 = tmem + C::TM_SFA1 + a1_bar[j] * 8;
#pragma unroll
                  for (int c = 0; c < 2; ++c)
                    tw::tc_mma_nvf4(acc + h * 128, D64 | (a1_lo[j] + 2 * c), D64 | (w1_lo + 2 * c), IDESC_128,
                                    t_sfa1 + 4 * c, t_sfw1 + 4 * c, 1u);
                }
                tw::tc_commit(emptyW1 + sw);
                if (++sw == C::W1_SLOTS) { sw = 0; pw ^= 1; }
              }
            }
            if (p.cross) {
#pragma unroll
              for (int j = 0; j < 2; ++j)
                if ((ab >> j) & 1u) tw::tc_commit(emptyA1 + a1_bar[j]);
            }
          }
          tw::tc_commit(emptyS + s);
          if (++s == C::STAGES) { s = 0; ph ^= 1; }
          abits >>= 2;
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) wbits[h] >>= 2;
        }
        if (ok) tw::tc_commit(accFull + stage);
        tw::mbar_arrive(tabEmpty + tsl);
        if (++tsl == C::TAB_SLOTS) { tsl = 0; tph ^= 1; }
      }
    }
  } else if (warp == 4 || warp == 5) {
    // ------------------------------------------------------------------ scale copies smem -> TMEM
    // Issuing a tcgen05.cp costs its thread tens of cycles and a K256 step needs 4 * (1 + BN/128)
    // of them plus two per repair unit, so they are issued by two threads of their own instead of
    // the MMA issuer: thread 0 takes K64 slices {0,1} of the base stage and the A1 units, thread 1
    // slices {2,3} and the W1 units. Every smem stage / unit slot owns a TMEM scale region, which is
    // free again whenever that stage or slot was reloaded (its previous MMAs had finished by then).
    if (lane == 0) {
      const int c = warp - 4;
      constexpr uint64_t DSF = (uint64_t(1) << 46) | (uint64_t(128 >> 4) << 32);
      const uint32_t smem_u = tw::smem_u32(smem);
      const uint32_t sf0_base = (smem_u + C::OFF_SF0) >> 4;
      const uint32_t usf_base = (smem_u + (c == 0 ? C::OFF_SFA1 : C::OFF_SFW1)) >> 4;
      const uint32_t t_usf = tmem + (c == 0 ? C::TM_SFA1 : C::TM_SFW1);
      uint64_t* const unit_full = c == 0 ? fullA1 : fullW1;
      uint64_t* const unit_ready = c == 0 ? usfA : usfW;
      const uint32_t unit_slots = c == 0 ? C::A1_SLOTS : C::W1_SLOTS;
      uint32_t s = 0, ph = 0, su = 0, pu = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
        const int n_rows = min(BN, p.n - (tile % p.tiles_n) * BN);
        const TermTable<BN>& tab = table(it);
        ok = tw::mbar_wait(tabFull + it % C::TAB_SLOTS, (it / C::TAB_SLOTS) & 1, abort_flag);
        uint32_t bits[C::HALVES] = {};
        for (int st = 0; st < steps && ok; ++st) {
          const int kb0 = 2 * st, nq = p.kb - kb0 >= 2 ? 4 : 2;
          if ((kb0 & 31) == 0) {
            if (c == 0) bits[0] = tab.a1bits[kb0 >> 5];
            else {
#pragma unroll
              for (int h = 0; h < C::HALVES; ++h) bits[h] = tab.w1bits[h][kb0 >> 5];
            }
          }
          // the stage was reloaded only after the MMAs of its previous use finished, so its region is free
          ok = tw::mbar_wait(fullS + s, ph, abort_flag);
          if (!ok) break;
          const uint32_t sf_lo = sf0_base + s * (C::STAGE_SF >> 4);
          const uint32_t t_sfa0 = tmem + C::TM_SFA0 + s * 16, t_sfb0 = tmem + C::TM_SFB0 + s * 16 * C::HALVES;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int q = 2 * c + i;
            if (q < nq) {
              tw::tc_copy_scales(t_sfa0 + 4 * q, DSF | (sf_lo + q * 32));
#pragma unroll
              for (int h = 0; h < C::HALVES; ++h)
                if (h * 128 < n_rows)
                  tw::tc_copy_scales(t_sfb0 + 4 * C::HALVES * q + 4 * h, DSF | (sf_lo + (1 + h) * 128 + q * 32));
            }
          }
          tw::tc_commit(sfFull + s);
          if (++s == C::STAGES) { s = 0; ph ^= 1; }
          // units of this step, in the order the MMA issuer consumes them
          int count = 0;
          if (c == 0) count = __popc(bits[0] & 3u);
          else {
#pragma unroll
            for (int h = 0; h < C::HALVES; ++h) count += __popc(bits[h] & 3u);
          }
          for (int u = 0; u < count && ok; ++u) {
            ok = tw::mbar_wait(unit_full + su, pu, abort_flag);
            if (!ok) break;
            const uint32_t lo = usf_base + su * (SF_ATOM >> 4);
            tw::tc_copy_scales(t_usf + su * 8, DSF | lo);
            tw::tc_copy_scales(t_usf + su * 8 + 4, DSF | (lo + 32));
            tw::tc_commit(unit_ready + su);
            if (++su == unit_slots) { su = 0; pu ^= 1; }
          }
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) bits[h] >>= 2;
        }
        tw::mbar_arrive(tabEmpty + it % C::TAB_SLOTS);
      }
    }
  } else if (warp >= C::FIRST_EPI_WARP) {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;                              // TMEM lane quadrant this warp may read
    const int group = (warp - C::FIRST_EPI_WARP) >> 2;      // column group
    const float alpha = __ldg(p.alpha);
    uint32_t it = 0;
    for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++it) {
      const int mbi = tile / p.tiles_n, nt = tile % p.tiles_n;
      const uint32_t stage = it % C::ACC_STAGES, aph = (it / C::ACC_STAGES) & 1;
      if (!tw::mbar_wait_warp(accFull + stage, aph, abort_flag)) break;
      tw::tc_fence_after();
      const uint32_t t_base = tmem + ((uint32_t)(quad * 32) << 16) + C::TM_ACC + stage * BN + group * C::EPI_COLS;
      const int row = mbi * 128 + quad * 32 + lane;
      const int col = nt * BN + group * C::EPI_COLS;
      __nv_bfloat16* dst = p.out + (size_t)row * p.n + col;
      const bool store = row < p.m && col < p.n;
      // 64 columns per round: two back-to-back TMEM loads, one wait; the TMEM stage is handed back
      // after the last round's loads, before that round is converted and stored
#pragma unroll
      for (int round = 0; round < C::EPI_COLS / 64; ++round) {
        uint32_t r[2][32];
        tw::tmem_load_32x32(t_base + round * 64, r[0]);
        tw::tmem_load_32x32(t_base + round * 64 + 32, r[1]);
        tw::tmem_load_wait();
        if (round == C::EPI_COLS / 64 - 1) {
          tw::tc_fence_before();
          __syncwarp();
          if (lane == 0) tw::mbar_arrive(accEmpty + stage);
        }
        if (store) {
#pragma unroll
          for (int part = 0; part < 2; ++part) {
#pragma unroll
            for (int v = 0; v < 2; ++v) {                   // 16 columns = 32 bytes per store
              uint32_t w[8];
              uint32_t bw[8] = {};
              if (p.bias) {
                const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col + round * 64 + part * 32 + v * 16);
                const uint4 b0 = __ldg(bp), b1 = __ldg(bp + 1);
                bw[0] = b0.x; bw[1] = b0.y; bw[2] = b0.z; bw[3] = b0.w; bw[4] = b1.x; bw[5] = b1.y; bw[6] = b1.z; bw[7] = b1.w;
              }
#pragma unroll
              for (int q = 0; q < 8; ++q) {
                const float lo = __fmaf_rn(__uint_as_float(r[part][16 * v + 2 * q]), alpha, tw::bf16_bits_to_float(bw[q] & 0xffffu));
                const float hi = __fmaf_rn(__uint_as_float(r[part][16 * v + 2 * q + 1]), alpha, tw::bf16_bits_to_float(bw[q] >> 16));
                __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
                w[q] = *reinterpret_cast<uint32_t*>(&b2);
              }
              tw::store_256(dst + round * 64 + part * 32 + v * 16, w);
            }
          }
        }
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

bool make_map(CUtensorMap* map, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides,
              const cuuint32_t* box, CUtensorMapSwizzle swz) {
  cuuint32_t ones[3] = {1, 1, 1};
  return encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box,
                     ones, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, bool DEEP>
int launch(int m, int n, int k, const void* a_codes, const void* w_codes, const void* sfa, const void* sfb, void* out,
           const float* alpha, void* workspace, cudaStream_t stream, const TwRepairIO* io, int sms, int dev) {
  using C = Cfg<BN, DEEP>;
  CUtensorMap tm_a0, tm_a1, tm_w0, tm_w1;
  const int planes = io->na > 0 ? 2 : 1;
  {
    // activation codes [planes, mp, k/2]: K256 boxes for the base plane, K128 boxes for residual blocks
    cuuint64_t dims[3] = {(cuuint64_t)k / 2, (cuuint64_t)io->mp, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)k / 2, (cuuint64_t)io->mp * (k / 2)};
    cuuint32_t box0[3] = {128, 128, 1}, box1[3] = {64, 128, 1};
    if (!make_map(&tm_a0, 3, a_codes, dims, strides, box0, CU_TENSOR_MAP_SWIZZLE_128B)) return TW_ERR_TENSOR_MAP;
    if (!make_map(&tm_a1, 3, a_codes, dims, strides, box1, CU_TENSOR_MAP_SWIZZLE_64B)) return TW_ERR_TENSOR_MAP;
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)k / 2, (cuuint64_t)n};
    cuuint64_t strides[1] = {(cuuint64_t)k / 2};
    cuuint32_t box[2] = {128, (cuuint32_t)BN};
    if (!make_map(&tm_w0, 2, w_codes, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return TW_ERR_TENSOR_MAP;
  }
  {
    const bool has = io->hasw != 0;
    cuuint64_t dims[2] = {64, (cuuint64_t)(has ? (size_t)io->bank_blocks * 128 : 128)};
    cuuint64_t strides[1] = {64};
    cuuint32_t box[2] = {64, 128};
    if (!make_map(&tm_w1, 2, has ? (const void*)io->wr : w_codes, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B))
      return TW_ERR_TENSOR_MAP;
  }
  Params p{};
  p.sfa0 = static_cast<const uint8_t*>(sfa);
  p.sfa1 = io->a1s_swz;
  p.sfb0 = static_cast<const uint8_t*>(sfb);
  p.sfbw = io->wrs_swz;
  p.wi = io->wi; p.off = io->off; p.wloc = io->wloc; p.mask = io->mask;
  p.alpha = alpha;
  p.bias = static_cast<const __nv_bfloat16*>(io->bias);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = static_cast<int*>(workspace);
  p.m = m; p.mp = io->mp; p.n = n; p.k = k; p.na = io->na; p.hasw = io->hasw; p.cross = io->cross;
  p.shared = io->shared; p.dense = io->dense; p.mask_per_n = io->mask_per_n;
  p.kb = k / 128; p.nb = n / 128; p.mb = (m + 127) / 128;
  p.tiles_n = (n + BN - 1) / BN;
  p.tiles = p.mb * p.tiles_n;
  static std::atomic<bool> configured[64];       // the shared-memory opt-in is a per-device attribute of the function
  if (!configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(fused_kernel<BN, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
      return TW_ERR_LAUNCH;
    configured[dev].store(true, std::memory_order_release);
  }
  const int grid = p.tiles < sms ? p.tiles : sms;
  fused_kernel<BN, DEEP><<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(tm_a0, tm_a1, tm_w0, tm_w1, p);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

}  // namespace

extern "C" size_t tw_workspace(int, int, int) { return 256; }

extern "C" int tw_fused_tile_n(int n) { return n % 256 == 0 ? 256 : 128; }

extern "C" int tw_fused(int m, int n, int k, const void* a_codes, const void* w_codes, const void* sfa, const void* sfb,
                        void* out, const float* alpha, void* workspace, void* stream, const TwRepairIO* io) {
  if (!io || !a_codes || !w_codes || !sfa || !sfb || !out || !alpha || !workspace) return TW_ERR_ARGUMENT;
  if (m <= 0 || n <= 0 || k <= 0) return TW_ERR_ARGUMENT;
  if (n % 128 || k % 128) return TW_ERR_SHAPE;
  if (k / 128 > KB_MAX) return TW_ERR_TOO_LARGE;
  if (io->m != m || io->n != n || io->k != k || io->mp != (m + 15) / 16 * 16) return TW_ERR_SHAPE;
  if (io->na < 0 || io->na > k / 128) return TW_ERR_ARGUMENT;
  if (io->na > 0 && !io->a1s_swz) return TW_ERR_MISSING_SWIZZLED;
  if (io->na > 0 && (io->mask_per_n || io->na < k / 128) && !io->mask) return TW_ERR_ARGUMENT;
  if (io->hasw) {
    if (!io->wr || !io->wrs_swz) return TW_ERR_MISSING_SWIZZLED;
    if (io->bank_blocks <= 0) return TW_ERR_ARGUMENT;
    if (!io->dense && (!io->wi || !io->off)) return TW_ERR_ARGUMENT;
    if (io->shared && !io->wloc) return TW_ERR_ARGUMENT;
  }
  const uintptr_t align = (uintptr_t)a_codes | (uintptr_t)w_codes | (uintptr_t)sfa | (uintptr_t)sfb | (uintptr_t)out |
                          (uintptr_t)io->a1s_swz | (uintptr_t)io->wrs_swz | (uintptr_t)io->wr;
  // TMA bases and bulk copies: 16 bytes; bias rows are read as 16-byte vectors; output rows are written
  // with 32-byte stores
  if ((align & 15) || ((uintptr_t)io->bias & 15) || ((uintptr_t)out & 31)) return TW_ERR_ALIGNMENT;
  if (!encode_fn()) return TW_ERR_DRIVER;
  int dev = 0, sms = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TW_ERR_LAUNCH;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
  if (major != 10) return TW_ERR_ARCH;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (n % 256 == 0 && !io->mask_per_n) {
    // with W1 tiles and an A1 quota of at least half the K blocks the unit rings are the scarcer resource
    // (2x plan: +1 %), below that the third base stage is (1.5x plan: +1.3 %, base plan: +16 %)
    if (io->hasw && 2 * io->na >= k / 128) return launch<256, true>(m, n, k, a_codes, w_codes, sfa, sfb, out, alpha, workspace, s, io, sms, dev);
    return launch<256, false>(m, n, k, a_codes, w_codes, sfa, sfb, out, alpha, workspace, s, io, sms, dev);
  }
  return launch<128, false>(m, n, k, a_codes, w_codes, sfa, sfb, out, alpha, workspace, s, io, sms, dev);
}
