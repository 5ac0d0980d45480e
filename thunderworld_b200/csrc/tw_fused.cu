// Fused selective-repair GEMM for sm_100a.
//
//   out = alpha * ( A0 W0^T + A1 W0^T|a-support + A0 W1^T|w-tiles [+ A1 W1^T|both] )      bf16 [M,N]
//
// All operands are NVFP4 (E2M1 codes, one UE4M3 scale per 16 k). Every term is issued as
// tcgen05.mma kind::mxf4nvf4.block_scale into ONE fp32 accumulator in tensor memory; the epilogue
// scales by the device scalar alpha and rounds to bf16 once. Term structure follows the reference
// (thunderworld_fp4/_native.py:11-62; cutlass/repair_collective.cuh:117-132); what differs is the
// schedule. The K loop advances in steps of 256 (two blocks of the K128 repair lattice): a "base
// stage" holds A0 (128 x 128 B) and W0 (BN x 128 B) of the step with their scales; the repair
// operands of the same step (A1 blocks, W1 tiles: "units" of 128 x 64 B) arrive through a second
// ring and are multiplied against the resident base stage, so W0 is fetched once for A0 and A1,
// and A0 once for W0 and W1.
//
// CTA = one 128 x BN output tile at a time (persistent over tiles), warp-specialised. Every role
// runs as a whole, converged warp and elects one lane only around the asynchronous instructions
// (TMA, tcgen05.cp / .mma / .commit): issued from a divergent single-lane branch the same
// instructions cost the issuing thread tens of cycles each and the tensor pipe starves.
//   warp 0      producer of base stages (TMA, 128-byte swizzle; bulk copies of scale atoms)
//   warp 1      MMA issuer: scale copies smem -> TMEM (tcgen05.cp), MMAs, commits
//   warps 2, 6  producers of repair units (A1 blocks / W1 tiles; TMA, 64-byte swizzle)
//   warp 3      builds the per-tile term tables (A-support bits, W1 bank positions) ahead of use
//   warps 8-15  epilogue: TMEM -> registers -> bf16 -> global (32-byte stores)
// Tensor memory: two accumulators whose column ranges overlap by 64 ([0,256) and [192,448) for
// 256-wide tiles) plus 64 columns of scale factors. The epilogue of a tile drains the shared
// columns first and then tells the MMA issuer, so the next tile's MMAs run under the rest of the
// drain. tcgen05.cp and tcgen05.mma of one thread execute in issue order, so each scale region is
// single and is rewritten for the next step without a barrier.
// No cluster, no multicast.
#include <atomic>
#include <cuda.h>
#include "tw_common.cuh"
#include "../../include/twb200.h"

namespace {

constexpr int KB_MAX = 192;               // K <= 24576
constexpr int UNIT_TILE = 128 * 64;       // bytes of one 128-row x K128 code tile
constexpr int SF_ATOM = 1024;             // bytes of the scales of 128 rows x K128

// DEEP = true: the call issues repair terms; one base stage of the 256-wide tile is traded for the unit rings.
// Without repair terms (plain W4A4) the rings shrink to one unused slot each and the third base stage stays.
template <int BN, bool DEEP = false> struct Cfg {
  static constexpr int HALVES = BN / 128;
  static constexpr int STAGES = BN == 256 && DEEP ? 2 : 3;    // base stages (K256 of A0 and W0)
  static constexpr int A1_SLOTS = DEEP ? 3 : 1;               // A1 units
  static constexpr int W1_SLOTS = DEEP ? (BN == 256 ? 5 : 3) : 1;  // W1 units
  static constexpr int TAB_SLOTS = 3;                         // per-tile term tables built ahead
  static constexpr int EPI_WARPS = 8;
  static constexpr int FIRST_EPI_WARP = 8;                    // warps 0-3 and 6 are control roles, 4, 5, 7 idle
  static constexpr int EPI_GROUPS = EPI_WARPS / 4;            // column groups per lane quadrant
  static constexpr int EPI_COLS = BN / EPI_GROUPS;            // columns per epilogue warp
  static constexpr int EPI_ROUNDS = EPI_COLS / 64;
  static constexpr int THREADS = (FIRST_EPI_WARP + EPI_WARPS) * 32;
  static constexpr int A0_TILE = 128 * 128;                   // 128 rows x K256
  static constexpr int W0_TILE = BN * 128;
  static constexpr int STAGE_SF = (1 + HALVES) * 2 * SF_ATOM; // A0 scales then W0 scales per half
  // shared-memory carve-up (offsets from a 1024-aligned base)
  static constexpr int OFF_A0 = 0;
  static constexpr int OFF_W0 = OFF_A0 + STAGES * A0_TILE;
  static constexpr int OFF_A1 = OFF_W0 + STAGES * W0_TILE;
  static constexpr int OFF_W1 = OFF_A1 + A1_SLOTS * UNIT_TILE;
  static constexpr int EPI_BYTES = EPI_WARPS * 32 * 128;      // per epilogue warp: 32 rows x 64 bf16 columns, staged for a TMA store
  static constexpr int OFF_EPI = OFF_W1 + W1_SLOTS * UNIT_TILE;
  static constexpr int OFF_SF0 = OFF_EPI + EPI_BYTES;
  static constexpr int OFF_SFA1 = OFF_SF0 + STAGES * STAGE_SF;
  static constexpr int OFF_SFW1 = OFF_SFA1 + A1_SLOTS * SF_ATOM;
  static constexpr int OFF_TAB = OFF_SFW1 + W1_SLOTS * SF_ATOM;
  static constexpr int TAB_BYTES = HALVES * KB_MAX * 4 + (HALVES + 1) * (KB_MAX / 32) * 4;
  static constexpr int OFF_BAR = OFF_TAB + TAB_SLOTS * TAB_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + A1_SLOTS + W1_SLOTS + 2 * TAB_SLOTS + 2 + 1;
  static constexpr int SMEM_BYTES = OFF_BAR + NUM_BARS * 8 + 64 + 1024;  // + alignment slack
  // tensor-memory columns: two accumulators (tile i uses accumulator i & 1) that share the columns
  // [ACC_STRIDE, BN), then the scale regions
  static constexpr int ACC_STRIDE = BN == 256 ? 192 : 128;
  static constexpr int TM_SF = ACC_STRIDE + BN;                          // 448 (256 for 128-wide tiles)
  static constexpr int TM_SFA0 = TM_SF;                                  // 16 columns: A0 scales of the step
  static constexpr int TM_SFB0 = TM_SFA0 + 16;                           // 16 * HALVES: W0 scales of the step
  static constexpr int TM_SFA1 = TM_SFB0 + 16 * HALVES;                  // 8: the A1 block being multiplied
  static constexpr int TM_SFW1 = TM_SFA1 + 8;                            // 8: the W1 tile being multiplied
  static constexpr int TM_COLS = 512;
  static_assert(TM_SFW1 + 8 <= TM_COLS, "tensor memory budget");
  // a step is issued only when all its units have landed, so the rings must hold the units of one step
  static_assert(!DEEP || (A1_SLOTS >= 2 && W1_SLOTS >= 2 * HALVES), "unit rings hold at least one step");
};
static_assert(Cfg<256>::SMEM_BYTES <= 232448 && Cfg<256, true>::SMEM_BYTES <= 232448 && Cfg<128>::SMEM_BYTES <= 232448 &&
              Cfg<128, true>::SMEM_BYTES <= 232448,
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
  int act;                  // nonzero: tanh-form GELU of the bf16-rounded result, rounded to bf16 again
  float* stats;             // with act, optional: {max|out| / 2688, max|out|}
  unsigned* scratch;        // two zeroed words: running maximum (float bits), CTA ticket
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
             const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
             const __grid_constant__ CUtensorMap tm_out, const Params p) {
  using C = Cfg<BN, DEEP>;
  extern __shared__ uint8_t smem_raw[];
  // aligned by pointer arithmetic on the __shared__ array (not through an integer cast), so that the compiler
  // keeps the address space and emits shared-memory loads and stores instead of generic ones
  uint8_t* smem = smem_raw + ((1024u - (tw::smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* fullS = bars;                       // a step's operands (base stage and its repair units) have landed
  uint64_t* emptyS = fullS + C::STAGES;         // the MMAs that read the base stage have completed
  uint64_t* emptyA1 = emptyS + C::STAGES;       // the MMAs that read an A1 / W1 unit slot have completed
  uint64_t* emptyW1 = emptyA1 + C::A1_SLOTS;
  uint64_t* tabFull = emptyW1 + C::W1_SLOTS;
  uint64_t* tabEmpty = tabFull + C::TAB_SLOTS;
  uint64_t* accFull = tabEmpty + C::TAB_SLOTS;  // [2]: every term of the tile in accumulator a has been accumulated
  uint64_t* sharedFree = accFull + 2;           // the epilogue has read the columns both accumulators share
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sharedFree + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto table = [&](uint32_t i) -> TermTable<BN>& {
    return *reinterpret_cast<TermTable<BN>*>(smem + C::OFF_TAB + (i % C::TAB_SLOTS) * C::TAB_BYTES);
  };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int steps = (p.kb + 1) / 2;             // K256 steps; the last one may hold a single K128 block

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::STAGES; ++i) { tw::mbar_init(fullS + i, 3); tw::mbar_init(emptyS + i, 1); }
    for (int i = 0; i < C::A1_SLOTS; ++i) tw::mbar_init(emptyA1 + i, 1);
    for (int i = 0; i < C::W1_SLOTS; ++i) tw::mbar_init(emptyW1 + i, 1);
    for (int i = 0; i < C::TAB_SLOTS; ++i) { tw::mbar_init(tabFull + i, 1); tw::mbar_init(tabEmpty + i, 3); }
    tw::mbar_init(accFull, 1); tw::mbar_init(accFull + 1, 1);
    tw::mbar_init(sharedFree, C::EPI_WARPS);
    *abort_flag = 0;
    tw::fence_barrier_init();
    tw::tma_prefetch_desc(&tm_a0); tw::tma_prefetch_desc(&tm_a1);
    tw::tma_prefetch_desc(&tm_w0); tw::tma_prefetch_desc(&tm_w1); tw::tma_prefetch_desc(&tm_out);
  }
  if (warp == 1) { tw::tmem_alloc(tmem_slot, C::TM_COLS); tw::tmem_relinquish(); }
  tw::tc_fence_before();
  __syncthreads();
  tw::tc_fence_after();
  // The kernel owns all 512 columns of the SM's tensor memory, so the allocation starts at lane 0, column 0;
  // using the constant keeps every tensor-memory address of the MMA issuer a compile-time value. A different
  // answer (it would mean another allocation is live on this SM) is reported, not ignored.
  if (*tmem_slot != 0u) *abort_flag = 1;
  constexpr uint32_t tmem = 0u;

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
    uint32_t s = 0, ph = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x) {
      const int mbi = tile / p.tiles_n, nt = tile % p.tiles_n;
      const int n_rows = min(BN, p.n - nt * BN);            // 128 or BN
      for (int st = 0; st < steps && ok; ++st) {
        const int kb0 = 2 * st, nk = min(2, p.kb - kb0);     // K128 blocks in this step
        ok = tw::mbar_wait_all(emptyS + s, ph ^ 1, abort_flag);
        if (!ok) break;
        if (tw::elect_one()) {
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
        __syncwarp();
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 2 || warp == 6) {
    // ------------------------------------------------------------------ producers of repair units
    // Warp 2 loads the A1 blocks, warp 6 the W1 tiles of every step, in the order the MMA issuer consumes
    // them. Their bytes complete on the step's stage barrier (it counts three arrivals: the base producer
    // and these two, with or without units), so the issuer waits once per step; slots are recycled through
    // their own barriers, which the issuer commits after the unit's last MMA.
    const bool do_a = warp == 2;
    uint32_t s = 0, ph = 0, sa = 0, pa = 0, sw = 0, pw = 0, it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
      const int mbi = tile / p.tiles_n;
      const TermTable<BN>& tab = table(it);
      ok = tw::mbar_wait_all(tabFull + it % C::TAB_SLOTS, (it / C::TAB_SLOTS) & 1, abort_flag);
      uint32_t abits = 0, wbits[C::HALVES] = {};
      for (int st = 0; st < steps && ok; ++st) {
        const int kb0 = 2 * st;
        if ((kb0 & 31) == 0) {
          abits = tab.a1bits[kb0 >> 5];
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) wbits[h] = tab.w1bits[h][kb0 >> 5];
        }
        uint32_t mine = 0;                                     // bit 2j + h: unit of block j (half h for W1)
        if (do_a) mine = (abits & 1u) | ((abits & 2u) << 1);
        else {
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) mine |= ((wbits[h] & 1u) << h) | ((wbits[h] & 2u) << (1 + h));
        }
        ok = tw::mbar_wait_all(emptyS + s, ph ^ 1, abort_flag);    // the stage barrier is in its next phase
        if (!ok) break;
        if (tw::elect_one()) {
          if (mine) tw::mbar_expect_tx(fullS + s, (uint32_t)__popc(mine) * (UNIT_TILE + SF_ATOM));
          else tw::mbar_arrive(fullS + s);
        }
        __syncwarp();
#pragma unroll 1
        while (mine && ok) {
          const uint32_t u = __ffs(mine) - 1;
          mine &= mine - 1;
          const int kb = kb0 + (int)(u >> 1);
          if (do_a) {
            ok = tw::mbar_wait_all(emptyA1 + sa, pa ^ 1, abort_flag);
            if (!ok) break;
            if (tw::elect_one()) {
              tw::tma_load_3d(smem + C::OFF_A1 + sa * UNIT_TILE, &tm_a1, kb * 64, mbi * 128, 1, fullS + s);
              tw::bulk_load(smem + C::OFF_SFA1 + sa * SF_ATOM, p.sfa1 + ((size_t)mbi * p.kb + kb) * SF_ATOM, SF_ATOM, fullS + s);
            }
            __syncwarp();
            if (++sa == C::A1_SLOTS) { sa = 0; pa ^= 1; }
          } else {
            const int loc = tab.w1loc[u & 1u][kb];
            ok = tw::mbar_wait_all(emptyW1 + sw, pw ^ 1, abort_flag);
            if (!ok) break;
            if (tw::elect_one()) {
              tw::tma_load_2d(smem + C::OFF_W1 + sw * UNIT_TILE, &tm_w1, 0, loc * 128, fullS + s);
              tw::bulk_load(smem + C::OFF_SFW1 + sw * SF_ATOM, p.sfbw + (size_t)loc * SF_ATOM, SF_ATOM, fullS + s);
            }
            __syncwarp();
            if (++sw == C::W1_SLOTS) { sw = 0; pw ^= 1; }
          }
        }
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
        abits >>= 2;
#pragma unroll
        for (int h = 0; h < C::HALVES; ++h) wbits[h] >>= 2;
      }
      if (tw::elect_one()) tw::mbar_arrive(tabEmpty + it % C::TAB_SLOTS);
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks the schedule (waits are warp-wide, every branch is warp-uniform); one elected
    // lane issues all tcgen05 operations of a step in one go: scale copies and MMAs of the base stage, then
    // of its repair units, then the commits that release the stage and the unit slots. The stage barrier
    // of the next step is polled before the current step is issued, so its latency hides behind the issue.
    // Descriptors are a constant high word plus (address >> 4).
    bool ok = true;
    constexpr uint32_t IDESC_FULL = tw::make_idesc_nvf4(128, BN);
    constexpr uint32_t IDESC_128 = tw::make_idesc_nvf4(128, 128);
    constexpr uint64_t D128 = (uint64_t(1) << 46) | (uint64_t(2) << 61) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 16);
    constexpr uint64_t D64 = (uint64_t(1) << 46) | (uint64_t(4) << 61) | (uint64_t(512 >> 4) << 32) | (uint64_t(1) << 16);
    constexpr uint64_t DSF = (uint64_t(1) << 46) | (uint64_t(128 >> 4) << 32);
    const uint32_t smem_u = tw::smem_u32(smem);
    const uint32_t a0_base = (smem_u + C::OFF_A0) >> 4, w0_base = (smem_u + C::OFF_W0) >> 4;
    const uint32_t a1_base = (smem_u + C::OFF_A1) >> 4, w1_base = (smem_u + C::OFF_W1) >> 4;
    const uint32_t sf0_base = (smem_u + C::OFF_SF0) >> 4;
    const uint32_t sfa1_base = (smem_u + C::OFF_SFA1) >> 4, sfw1_base = (smem_u + C::OFF_SFW1) >> 4;
    const uint32_t t_sfa0 = tmem + C::TM_SFA0, t_sfb0 = tmem + C::TM_SFB0;
    const uint32_t t_sfa1 = tmem + C::TM_SFA1, t_sfw1 = tmem + C::TM_SFW1;
    uint32_t s = 0, ph = 0;                  // base stage slot / phase
    uint32_t sa = 0, sw = 0;                 // next unit slots
    uint32_t it = 0, tsl = 0, tph = 0;       // tile counter, table slot / phase
    bool ready = tw::mbar_test_wait(fullS, 0);
    for (int tile = blockIdx.x; tile < p.tiles && ok; tile += gridDim.x, ++it) {
      const int nt = tile % p.tiles_n;
      const TermTable<BN>& tab = *reinterpret_cast<const TermTable<BN>*>(smem + C::OFF_TAB + tsl * C::TAB_BYTES);
      const int n_rows = min(BN, p.n - nt * BN);
      const uint32_t idesc_base = n_rows == BN ? IDESC_FULL : IDESC_128;
      ok = tw::mbar_wait_all(tabFull + tsl, tph, abort_flag);
      // the previous tile's epilogue has read the columns this accumulator shares with its own
      // (its tcgen05.ld have completed - tcgen05.wait::ld - before it arrives on the barrier, so the MMAs
      // issued below cannot overtake them)
      if (ok && it > 0) ok = tw::mbar_wait_all(sharedFree, (it - 1) & 1, abort_flag);
      const uint32_t acc = tmem + (it & 1) * C::ACC_STRIDE;
      uint32_t abits = 0, wbits[C::HALVES] = {};
      for (int st = 0; st < steps && ok; ++st) {
        const int kb0 = 2 * st;
        const int nq = p.kb - kb0 >= 2 ? 4 : 2;                  // K64 slices in this step
        if ((kb0 & 31) == 0) {
          abits = tab.a1bits[kb0 >> 5];
#pragma unroll
          for (int h = 0; h < C::HALVES; ++h) wbits[h] = tab.w1bits[h][kb0 >> 5];
        }
        // units of this step in issue order: bit 3j = A1 of block j, bit 3j + 1 + h = W1 tile (block j, half h)
        uint32_t units = (abits & 1u) | ((abits & 2u) << 2);
#pragma unroll
        for (int h = 0; h < C::HALVES; ++h) units |= ((wbits[h] & 1u) << (1 + h)) | ((wbits[h] & 2u) << (3 + h));
        // operands arrive through the async proxy (TMA) and are consumed by it (tcgen05): no fence is needed
        if (!ready) ok = tw::mbar_wait_all(fullS + s, ph, abort_flag);
        if (!ok) break;
        {
          const uint32_t sn = s + 1 == C::STAGES ? 0 : s + 1;
          ready = tw::mbar_test_wait(fullS + sn, sn == 0 ? ph ^ 1 : ph);
        }
        const uint32_t a0_lo = a0_base + s * (C::A0_TILE >> 4), w0_lo = w0_base + s * (C::W0_TILE >> 4);
        const uint32_t sf_lo = sf0_base + s * (C::STAGE_SF >> 4);
        if (tw::elect_one()) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (q < nq) {
              tw::tc_copy_scales(t_sfa0 + 4 * q, DSF | (sf_lo + q * 32));
#pragma unroll
              for (int h = 0; h < C::HALVES; ++h)
                if (h * 128 < n_rows)
                  tw::tc_copy_scales(t_sfb0 + 4 * C::HALVES * q + 4 * h, DSF | (sf_lo + (1 + h) * 128 + q * 32));
            }
          }
#pragma unroll
          for (int q = 0; q < 4; ++q)                              // A0 W0
            if (q < nq)
              tw::tc_mma_nvf4(acc, D128 | (a0_lo + 2 * q), D128 | (w0_lo + 2 * q), idesc_base, t_sfa0 + 4 * q,
                              t_sfb0 + 4 * C::HALVES * q, (st | q) != 0);
          // Repair terms of the two K128 blocks of this step, block by block: A1 W0, then per W1 tile A0 W1
          // (128-column MMAs into the matching half of the accumulator) and, with `cross`, A1 W1. One rolled
          // loop over the units that exist: the instruction footprint of a step stays small, which matters
          // because a taken branch over a long unrolled body costs this warp an instruction-cache miss.
          uint32_t todo = units, la = sa, lw = sw, a1_lo = 0;
#pragma unroll 1
          while (todo) {
            const uint32_t u = __ffs(todo) - 1;
            todo &= todo - 1;
            const uint32_t j = u >= 3 ? 1u : 0u, t = u - 3 * j;
            if (t == 0) {                                          // A1 block j against the resident W0 stage
              a1_lo = a1_base + la * (UNIT_TILE >> 4);
              const uint32_t usf = sfa1_base + la * (SF_ATOM >> 4);
              const uint32_t b_lo = w0_lo + 4 * j, sfb = t_sfb0 + 8 * C::HALVES * j;
              tw::tc_copy_scales(t_sfa1, DSF | usf);
              tw::tc_copy_scales(t_sfa1 + 4, DSF | (usf + 32));
              tw::tc_mma_nvf4(acc, D64 | a1_lo, D128 | b_lo, idesc_base, t_sfa1, sfb, 1u);
              tw::tc_mma_nvf4(acc, D64 | (a1_lo + 2), D128 | (b_lo + 2), idesc_base, t_sfa1 + 4, sfb + 4 * C::HALVES, 1u);
              // without a cross term nothing reads the block again
              if (!p.cross) tw::tc_commit(emptyA1 + la);
              if (++la == C::A1_SLOTS) la = 0;
            } else {                                               // W1 tile (block j, half t - 1) against A0
              const uint32_t w1_lo = w1_base + lw * (UNIT_TILE >> 4), usf = sfw1_base + lw * (SF_ATOM >> 4);
              const uint32_t a_lo = a0_lo + 4 * j, sfa = t_sfa0 + 8 * j, d = acc + (t - 1) * 128;
              tw::tc_copy_scales(t_sfw1, DSF | usf);
              tw::tc_copy_scales(t_sfw1 + 4, DSF | (usf + 32));
              tw::tc_mma_nvf4(d, D128 | a_lo, D64 | w1_lo, IDESC_128, sfa, t_sfw1, 1u);
              tw::tc_mma_nvf4(d, D128 | (a_lo + 2), D64 | (w1_lo + 2), IDESC_128, sfa + 4, t_sfw1 + 4, 1u);
              if (p.cross && ((units >> (3 * j)) & 1u)) {
                tw::tc_mma_nvf4(d, D64 | a1_lo, D64 | w1_lo, IDESC_128, t_sfa1, t_sfw1, 1u);
                tw::tc_mma_nvf4(d, D64 | (a1_lo + 2), D64 | (w1_lo + 2), IDESC_128, t_sfa1 + 4, t_sfw1 + 4, 1u);
              }
              tw::tc_commit(emptyW1 + lw);
              if (++lw == C::W1_SLOTS) lw = 0;
            }
          }
          if (p.cross && (units & 9u)) {                           // a cross term may have read them last
            tw::tc_commit(emptyA1 + sa);
            if ((units & 9u) == 9u) tw::tc_commit(emptyA1 + (sa + 1 == C::A1_SLOTS ? 0 : sa + 1));
          }
          tw::tc_commit(emptyS + s);
        }
        __syncwarp();
        // ring positions advance by at most one ring length per step: a conditional subtract, not a modulo (this
        // warp's instruction stream is the kernel's critical path)
        sa += __popc(units & 9u);
        if (sa >= (uint32_t)C::A1_SLOTS) sa -= C::A1_SLOTS;
        sw += __popc(units & 54u);
        if (sw >= (uint32_t)C::W1_SLOTS) sw -= C::W1_SLOTS;
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
        abits >>= 2;
#pragma unroll
        for (int h = 0; h < C::HALVES; ++h) wbits[h] >>= 2;
      }
      if (tw::elect_one()) {
        if (ok) tw::tc_commit(accFull + (it & 1));
        tw::mbar_arrive(tabEmpty + tsl);
      }
      __syncwarp();
      if (++tsl == C::TAB_SLOTS) { tsl = 0; tph ^= 1; }
    }
  } else if (warp >= C::FIRST_EPI_WARP) {
    // ------------------------------------------------------------------ epilogue
    // TMEM -> registers -> bf16 -> this warp's staging tile in shared memory (32 rows x 128 bytes, 128-byte
    // swizzle) -> one TMA store per 64 columns. Plain global stores of row-per-lane fragments touch 32 lines per
    // instruction and held this SM's load/store pipe for thousands of cycles per tile, behind which the MMA
    // issuer's own shared-memory and barrier operations queued; the bulk store leaves that pipe alone, writes
    // whole lines and clips rows beyond M by itself.
    const int quad = warp & 3;                              // TMEM lane quadrant this warp may read
    const int group = (warp - C::FIRST_EPI_WARP) >> 2;      // column group
    const float alpha = __ldg(p.alpha);
    uint8_t* stage = smem + C::OFF_EPI + (warp - C::FIRST_EPI_WARP) * 4096;
    uint8_t* my_row = stage + lane * 128;
    uint32_t it = 0;
    float peak = 0.f;                                       // max |activated output| of this lane's rows (rows < m only)
    for (int tile = blockIdx.x; tile < p.tiles; tile += gridDim.x, ++it) {
      const int mbi = tile / p.tiles_n, nt = tile % p.tiles_n;
      const uint32_t a = it & 1;
      if (!tw::mbar_wait_warp(accFull + a, (it >> 1) & 1, abort_flag)) break;
      tw::tc_fence_after();
      const uint32_t t_base = tmem + ((uint32_t)(quad * 32) << 16) + a * C::ACC_STRIDE + group * C::EPI_COLS;
      const int row0 = mbi * 128 + quad * 32;
      const int col = nt * BN + group * C::EPI_COLS;
      const bool live = col < p.n;                          // 128 columns of a 256-wide kernel never happen; kept for safety
      const bool in_m = row0 + lane < p.m;                  // rows beyond m are clipped by the store and excluded from the maximum
      // 64 columns per round: two back-to-back TMEM loads, one wait. Accumulator 0 shares its last 64
      // columns with accumulator 1's first 64, so the rounds of accumulator 0 run backwards: the shared
      // columns are read first and the MMA issuer is told before they are converted and stored.
#pragma unroll 1
      for (int i = 0; i < C::EPI_ROUNDS; ++i) {
        const int round = a == 0 ? C::EPI_ROUNDS - 1 - i : i;
        uint32_t r[2][32];
        tw::tmem_load_32x32(t_base + round * 64, r[0]);
        tw::tmem_load_32x32(t_base + round * 64 + 32, r[1]);
        tw::tmem_load_wait();
        if (i == 0) {
          tw::tc_fence_before();
          __syncwarp();
          if (lane == 0) tw::mbar_arrive(sharedFree);
        }
        // the previous store of this warp has finished reading the staging tile
        if (lane == 0) tw::bulk_store_wait_read();
        __syncwarp();
#pragma unroll
        for (int part = 0; part < 2; ++part) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {                     // 8 columns = 16 bytes per shared-memory store
            uint32_t bw[4] = {};
            if (p.bias) {
              const uint4 b0 = __ldg(reinterpret_cast<const uint4*>(p.bias + col + round * 64 + part * 32 + v * 8));
              bw[0] = b0.x; bw[1] = b0.y; bw[2] = b0.z; bw[3] = b0.w;
            }
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float lo = __fmaf_rn(__uint_as_float(r[part][8 * v + 2 * q]), alpha, tw::bf16_bits_to_float(bw[q] & 0xffffu));
              const float hi = __fmaf_rn(__uint_as_float(r[part][8 * v + 2 * q + 1]), alpha, tw::bf16_bits_to_float(bw[q] >> 16));
              __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
              if (p.act) {
                // the activation sees the bf16 value an unfused call would have stored, and is rounded once more
                b2 = __floats2bfloat162_rn(tw::gelu_tanh(__low2float(b2)), tw::gelu_tanh(__high2float(b2)));
                if (in_m) peak = fmaxf(peak, fmaxf(fabsf(__low2float(b2)), fabsf(__high2float(b2))));
              }
              w[q] = *reinterpret_cast<uint32_t*>(&b2);
            }
            const int chunk = part * 4 + v;                 // 16-byte chunk of the 128-byte row; swizzled by the row
            *reinterpret_cast<uint4*>(my_row + ((chunk ^ (lane & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        tw::fence_proxy_async();
        __syncwarp();
        if (lane == 0 && live) tw::tma_store_2d(&tm_out, stage, col + round * 64, row0);
      }
    }
    if (lane == 0) tw::bulk_store_wait_all();               // global writes are complete before the CTA exits
    if (p.act && p.stats) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
      // the bit pattern of a non-negative float orders like the float
      if (lane == 0) { atomicMax(p.scratch, __float_as_uint(peak)); __threadfence(); }
    }
  }

  tw::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(p.status, TW_ERR_TIMEOUT);
  if (threadIdx.x == 0 && p.act && p.stats) {
    // the last CTA to take a ticket publishes the tensor factor and clears the scratch for the next call
    __threadfence();
    if (atomicAdd(p.scratch + 1, 1u) == gridDim.x - 1) {
      __threadfence();
      const float top = __uint_as_float(atomicExch(p.scratch, 0u));
      p.stats[0] = top > 0.f ? __fdiv_rn(top, 2688.f) : 1.f;
      p.stats[1] = top;
      p.scratch[1] = 0u;
    }
  }
  if (warp == 1) { tw::tc_fence_after(); tw::tmem_dealloc(*tmem_slot, C::TM_COLS); }
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
  CUtensorMap tm_out;
  {
    // output bf16 [m, n]: boxes of 64 columns x 32 rows (one epilogue warp's staging tile); rows >= m are clipped
    cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)m};
    cuuint64_t strides[1] = {(cuuint64_t)n * 2};
    cuuint32_t box[2] = {64, 32}, ones[2] = {1, 1};
    if (encode_fn()(&tm_out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
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
  p.act = io->activation; p.stats = io->stats; p.scratch = io->stats_scratch;
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
  fused_kernel<BN, DEEP><<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(tm_a0, tm_a1, tm_w0, tm_w1, tm_out, p);
  return cudaGetLastError() == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}

}  // namespace

int tw_fused_pair_launch(int m, int n, int k, const void* a_codes, const void* w_codes, const void* sfa, const void* sfb,
                         void* out, const float* alpha, void* workspace, cudaStream_t stream, const TwRepairIO* io,
                         int sms, int dev);                              // tw_fused_pair.cu

extern "C" size_t tw_workspace(int, int, int) { return 256; }

extern "C" int tw_fused_tile_n(int n) { return n % 256 == 0 ? 256 : 128; }

extern "C" int tw_fused(int m, int n, int k, const void* a_codes, const void* w_codes, const void* sfa, const void* sfb,
                        void* out, const float* alpha, void* workspace, void* stream, const TwRepairIO* io) {
  if (!io || !a_codes || !w_codes || !sfa || !sfb || !out || !alpha || !workspace) return TW_ERR_ARGUMENT;
  if (m <= 0 || n <= 0 || k <= 0) return TW_ERR_ARGUMENT;
  if (n % 128 || k % 128) return TW_ERR_SHAPE;
  if (k / 128 > KB_MAX) return TW_ERR_TOO_LARGE;
  if (io->m != m || io->n != n || io->k != k || io->mp < (m + 15) / 16 * 16 || io->mp % 16) return TW_ERR_SHAPE;
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
  if (io->kernel < 0 || io->kernel > 3) return TW_ERR_ARGUMENT;
  if (io->activation != 0 && io->activation != TW_ACT_GELU_TANH) return TW_ERR_ARGUMENT;
  if ((io->stats && (!io->activation || !io->stats_scratch)) || (io->activation && io->kernel == 2)) return TW_ERR_ARGUMENT;
  // 256-wide tiles on CTA pairs (two row blocks per tile) unless the caller asks for the single-CTA kernel
  const bool pair_ok = n % 256 == 0 && !io->mask_per_n && m > 128;
  if (io->kernel == 2 && !pair_ok) return TW_ERR_SHAPE;
  // (measured on B200: the pair kernel does not beat the single-CTA kernel - both are bound by the rate at which
  // one thread can issue tcgen05 operations, and a pair has one issuing thread for two SMs - so it runs on request)
  if (pair_ok && io->kernel == 2)
    return tw_fused_pair_launch(m, n, k, a_codes, w_codes, sfa, sfb, out, alpha, workspace, s, io, sms, dev);
  const bool repair = io->na > 0 || io->hasw;
  if (n % 256 == 0 && !io->mask_per_n && io->kernel != 3) {
    if (repair) return launch<256, true>(m, n, k, a_codes, w_codes, sfa, sfb, out, alpha, workspace, s, io, sms, dev);
    return launch<256, false>(m, n, k, a_codes, w_codes, sfa, sfb, out, alpha, workspace, s, io, sms, dev);
  }
  if (repair) return launch<128, true>(m, n, k, a_codes, w_codes, sfa, sfb, out, alpha, workspace, s, io, sms, dev);
  return launch<128, false>(m, n, k, a_codes, w_codes, sfa, sfb, out, alpha, workspace, s, io, sms, dev);
}
