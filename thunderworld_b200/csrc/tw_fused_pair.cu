// Fused selective-repair GEMM for sm_100a on CTA pairs (tcgen05 cta_group::2).
//
//   out = alpha * ( A0 W0^T + A1 W0^T|a-support + A0 W1^T|w-tiles [+ A1 W1^T|both] )      bf16 [M,N]
//
// Same terms, operands and accumulation rule as the single-CTA kernel in tw_fused.cu (reference:
// thunderworld_fp4/_native.py:11-62, cutlass/repair_collective.cuh:117-132,
// tools/thor_handoff/sm110_repair_collective.cuh:87-169); what changes is that two CTAs of one cluster
// compute a 256 x 256 output tile together: every tcgen05.mma covers M = 256 (128 rows in each CTA's
// tensor memory), so the one thread that issues the MMAs of the pair feeds two tensor cores, and each
// CTA fetches only its own half of the W operands (128 of the 256 W0 rows, 64 of the 128 rows of a W1
// tile) - half the shared-memory traffic per issued FLOP.
//
// Rank r of the pair (cluster rank; 0 = leader) owns rows [ (2 pm + r) 128, +128 ) of the tile and the
// W0 rows [ nt 256 + r 128, +128 ). Per CTA and K256 step ("stage"): A0 own rows (16 KB, 128-byte swizzle),
// W0 own half (16 KB), A0 scales (2 KB), W0 scales of both halves (4 KB: every CTA needs the scales of
// all 256 columns in its tensor memory). Repair units of the step ride on the same stage barrier:
//   A1 block (kb): issued for the UNION of the two row blocks' supports, because one MMA spans both;
//                  the CTA whose block is not selected loads zeros (a TMA box outside the tensor), which
//                  contribute exactly 0 to its rows;
//   W1 tile (nb, kb): a 128-column MMA; each CTA holds 64 rows of the tile and all of its scales.
// Roles per CTA (whole, converged warps; one elected lane issues asynchronous instructions):
//   warp 0      producer of base stages          warp 2 / 6  producers of A1 / W1 units
//   warp 3      term tables, built ahead          warps 8-15  epilogue of the CTA's own 128 rows
//   warp 1      leader: MMA issuer of the pair (tcgen05.cp / .mma / .commit with cta_group::2; a commit
//               arrives on the same barrier in both CTAs)
//               peer: relay - waits for its own stage barrier and arrives on the leader's, so the leader
//               waits on one barrier per step for the operands of both CTAs
// Every load fills the issuing CTA's own shared memory from this GPU's memory; nothing is broadcast to the peer.
#include <atomic>
#include <cuda.h>
#include "tw_common.cuh"
#include "../../include/twb200.h"

namespace {

constexpr int KB_MAX = 192;               // K <= 24576
constexpr int UNIT_A = 128 * 64;          // bytes of an A1 unit: 128 rows x K128
constexpr int UNIT_W = 64 * 64;           // bytes of this CTA's half of a W1 unit: 64 rows x K128
constexpr int SF_ATOM = 1024;             // bytes of the scales of 128 rows x K128

struct PairCfg {
  static constexpr int STAGES = 4;
  static constexpr int A1_SLOTS = 4;
  static constexpr int W1_SLOTS = 6;
  static constexpr int TAB_SLOTS = 3;
  static constexpr int EPI_WARPS = 8;
  static constexpr int FIRST_EPI_WARP = 8;
  static constexpr int THREADS = (FIRST_EPI_WARP + EPI_WARPS) * 32;
  static constexpr int A0_TILE = 128 * 128;                   // own 128 rows x K256
  static constexpr int W0_TILE = 128 * 128;                   // own 128 of the tile's 256 W0 rows x K256
  static constexpr int STAGE_SF = 3 * 2 * SF_ATOM;            // A0 scales (own rows), W0 scales of both halves
  static constexpr int OFF_A0 = 0;
  static constexpr int OFF_W0 = OFF_A0 + STAGES * A0_TILE;
  static constexpr int OFF_A1 = OFF_W0 + STAGES * W0_TILE;
  static constexpr int OFF_W1 = OFF_A1 + A1_SLOTS * UNIT_A;
  static constexpr int OFF_SF0 = OFF_W1 + W1_SLOTS * UNIT_W;
  static constexpr int OFF_SFA1 = OFF_SF0 + STAGES * STAGE_SF;
  static constexpr int OFF_SFW1 = OFF_SFA1 + A1_SLOTS * SF_ATOM;
  static constexpr int OFF_TAB = OFF_SFW1 + W1_SLOTS * SF_ATOM;
  static constexpr int TAB_BYTES = 2 * KB_MAX * 4 + 4 * (KB_MAX / 32) * 4;
  static constexpr int OFF_BAR = OFF_TAB + TAB_SLOTS * TAB_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + A1_SLOTS + W1_SLOTS + 2 * TAB_SLOTS + 2 + 1;
  static constexpr int SMEM_BYTES = OFF_BAR + NUM_BARS * 8 + 64 + 1024;
  // tensor memory: two accumulators that share the columns [192, 256), then the scale regions
  static constexpr int ACC_STRIDE = 192;
  static constexpr int TM_SFA0 = 448, TM_SFB0 = 464, TM_SFA1 = 496, TM_SFW1 = 504, TM_COLS = 512;
  static_assert(A1_SLOTS >= 2 && W1_SLOTS >= 4, "unit rings hold at least one step");
};
static_assert(PairCfg::SMEM_BYTES <= 232448, "shared memory budget");

struct PairParams {
  const uint8_t *sfa0, *sfa1, *sfb0, *sfbw;
  const int *wi, *off, *wloc;
  const uint8_t* mask;
  const float* alpha;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;
  int* status;
  int m, n, k, na, hasw, cross, shared, dense;
  int kb, nb, mb, tiles_n, tiles;
};

// Per pair tile and CTA: one bit per kb for "an A1 block is issued" (union of the two row blocks) and "this
// CTA's own block is selected", one per (half, kb) for "a W1 tile exists", and the bank position of each tile.
struct PairTable {
  int w1loc[2][KB_MAX];
  uint32_t w1bits[2][KB_MAX / 32];
  uint32_t a_union[KB_MAX / 32];
  uint32_t a_own[KB_MAX / 32];
};
static_assert(sizeof(PairTable) == PairCfg::TAB_BYTES, "table size");

__device__ __forceinline__ void build_pair_table(PairTable& tab, const PairParams& p, int pm, int nt, int rank, int lane) {
  int begin[2], end[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int nb = nt * 2 + h;
    const bool use = p.hasw && !p.dense;
    begin[h] = use ? p.off[nb] : 0;
    end[h] = use ? p.off[nb + 1] : 0;
  }
  const int words = (p.kb + 31) / 32;
  for (int w = 0; w < words; ++w) {
    const int kb = w * 32 + lane;
    const bool in = kb < p.kb;
    bool sel[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int mbi = 2 * pm + r;
      sel[r] = in && mbi < p.mb && p.na > 0 && (p.na == p.kb || p.mask[(size_t)mbi * p.kb + kb] != 0);
    }
    const uint32_t uni = __ballot_sync(0xffffffffu, sel[0] || sel[1]);
    const uint32_t own = __ballot_sync(0xffffffffu, sel[rank]);
    if (lane == 0) { tab.a_union[w] = uni; tab.a_own[w] = own; }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const bool dense = in && p.hasw && p.dense;
      if (in) tab.w1loc[h][kb] = dense ? (nt * 2 + h) * p.kb + kb : -1;
      const uint32_t wb = __ballot_sync(0xffffffffu, dense);
      if (lane == 0) tab.w1bits[h][w] = wb;
    }
  }
  __syncwarp();
#pragma unroll
  for (int h = 0; h < 2; ++h)
    for (int s = begin[h] + lane; s < end[h]; s += 32) {
      const int kb = p.wi[s];
      tab.w1loc[h][kb] = p.shared ? p.wloc[s] : s;
      atomicOr(&tab.w1bits[h][kb >> 5], 1u << (kb & 31));
    }
  __syncwarp();
}

// ---- cluster / cta_group::2 primitives ---------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on the barrier at the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t rank) {
  asm volatile("{ .reg .b32 ra; mapa.shared::cluster.u32 ra, %0, %1;\n"
               "  mbarrier.arrive.release.cluster.shared::cluster.b64 _, [ra]; }" ::"r"(tw::smem_u32(bar)), "r"(rank) : "memory");
}
__device__ __forceinline__ void pair_tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tw::smem_u32(slot)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void pair_tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
// Arrives on `bar` (same offset) in both CTAs of the pair when every tcgen05 operation issued so far by this
// thread has completed (one barrier arrival delivered to both CTAs).
__device__ __forceinline__ void pair_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(tw::smem_u32(bar)), "h"((uint16_t)3) : "memory");
}
__device__ __forceinline__ void pair_copy_scales(uint32_t tmem_addr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc) : "memory");
}
// D[tmem, both CTAs] (+)= A[smem, 128 rows per CTA] * B[smem, N/2 rows per CTA]^T; K = 64.
__device__ __forceinline__ void pair_mma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                              uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "  tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p; }"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

__global__ void __launch_bounds__(PairCfg::THREADS, 1)
fused_pair_kernel(const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_a1,
                  const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1, const PairParams p) {
  using C = PairCfg;
  extern __shared__ uint8_t smem_raw[];
  // aligned by pointer arithmetic on the __shared__ array (not through an integer cast), so that the compiler
  // keeps the address space and emits shared-memory loads and stores instead of generic ones
  uint8_t* smem = smem_raw + ((1024u - (tw::smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* fullS = bars;                       // a step's operands have landed (leader: in both CTAs)
  uint64_t* emptyS = fullS + C::STAGES;         // the MMAs that read the base stage have completed
  uint64_t* emptyA1 = emptyS + C::STAGES;       // ... that read an A1 / W1 unit slot
  uint64_t* emptyW1 = emptyA1 + C::A1_SLOTS;
  uint64_t* tabFull = emptyW1 + C::W1_SLOTS;
  uint64_t* tabEmpty = tabFull + C::TAB_SLOTS;
  uint64_t* accFull = tabEmpty + C::TAB_SLOTS;  // [2]
  uint64_t* sharedFree = accFull + 2;           // leader: both epilogues have read the shared accumulator columns
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sharedFree + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto table = [&](uint32_t i) -> PairTable& {
    return *reinterpret_cast<PairTable*>(smem + C::OFF_TAB + (i % C::TAB_SLOTS) * C::TAB_BYTES);
  };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();      // 0 = leader
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int steps = (p.kb + 1) / 2;

  if (threadIdx.x == 0) {
    // leader: its own three producers and the peer's relay; peer: its own three producers
    for (int i = 0; i < C::STAGES; ++i) { tw::mbar_init(fullS + i, rank == 0 ? 4 : 3); tw::mbar_init(emptyS + i, 1); }
    for (int i = 0; i < C::A1_SLOTS; ++i) tw::mbar_init(emptyA1 + i, 1);
    for (int i = 0; i < C::W1_SLOTS; ++i) tw::mbar_init(emptyW1 + i, 1);
    for (int i = 0; i < C::TAB_SLOTS; ++i) { tw::mbar_init(tabFull + i, 1); tw::mbar_init(tabEmpty + i, 3); }
    tw::mbar_init(accFull, 1); tw::mbar_init(accFull + 1, 1);
    tw::mbar_init(sharedFree, 2 * C::EPI_WARPS);
    *abort_flag = 0;
    tw::fence_barrier_init();
    tw::tma_prefetch_desc(&tm_a0); tw::tma_prefetch_desc(&tm_a1);
    tw::tma_prefetch_desc(&tm_w0); tw::tma_prefetch_desc(&tm_w1);
  }
  // unit scale slots start as zeros: a CTA that loads zero codes for an unselected A1 block leaves the
  // slot's scales as they are, and whatever they are must decode to a finite value
  for (int i = threadIdx.x; i < (C::A1_SLOTS + C::W1_SLOTS) * SF_ATOM / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem + C::OFF_SFA1)[i] = make_uint4(0u, 0u, 0u, 0u);
  for (int i = threadIdx.x; i < C::STAGES * C::STAGE_SF / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem + C::OFF_SF0)[i] = make_uint4(0u, 0u, 0u, 0u);
  tw::fence_proxy_async();
  if (warp == 1) pair_tmem_alloc(tmem_slot, C::TM_COLS);
  tw::tc_fence_before();
  __syncthreads();
  cluster_sync_all();                            // barriers of both CTAs exist before anything arrives remotely
  tw::tc_fence_after();
  // The kernel owns all 512 columns of the SM's tensor memory, so the allocation starts at lane 0, column 0;
  // using the constant keeps every tensor-memory address of the MMA issuer a compile-time value. A different
  // answer (it would mean another allocation is live on this SM) is reported, not ignored.
  if (*tmem_slot != 0u) *abort_flag = 1;
  constexpr uint32_t tmem = 0u;

  if (warp == 3) {
    // ------------------------------------------------------------------ term tables, built ahead
    uint32_t it = 0;
    for (int tile = pair; tile < p.tiles; tile += pairs, ++it) {
      if (!tw::mbar_wait_warp(tabEmpty + it % C::TAB_SLOTS, ((it / C::TAB_SLOTS) & 1) ^ 1, abort_flag)) break;
      build_pair_table(table(it), p, tile / p.tiles_n, tile % p.tiles_n, (int)rank, lane);
      if (lane == 0) tw::mbar_arrive(tabFull + it % C::TAB_SLOTS);
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------------ producer of base stages
    uint32_t s = 0, ph = 0;
    bool ok = true;
    for (int tile = pair; tile < p.tiles && ok; tile += pairs) {
      const int mbi = 2 * (tile / p.tiles_n) + (int)rank, nt = tile % p.tiles_n;
      const bool rows = mbi < p.mb;                 // an odd number of row blocks leaves the last peer without rows
      for (int st = 0; st < steps && ok; ++st) {
        const int kb0 = 2 * st, nk = min(2, p.kb - kb0);
        ok = tw::mbar_wait_all(emptyS + s, ph ^ 1, abort_flag);
        if (!ok) break;
        if (tw::elect_one()) {
          // TMA always delivers the full box (out-of-range rows or K read as zero codes)
          tw::mbar_expect_tx(fullS + s, C::A0_TILE + C::W0_TILE + (uint32_t)((rows ? 1 : 0) + 2) * nk * SF_ATOM);
          tw::tma_load_3d(smem + C::OFF_A0 + s * C::A0_TILE, &tm_a0, kb0 * 64, mbi * 128, 0, fullS + s);
          tw::tma_load_2d(smem + C::OFF_W0 + s * C::W0_TILE, &tm_w0, kb0 * 64, nt * 256 + (int)rank * 128, fullS + s);
          uint8_t* sf = smem + C::OFF_SF0 + s * C::STAGE_SF;
          if (rows) tw::bulk_load(sf, p.sfa0 + ((size_t)mbi * p.kb + kb0) * SF_ATOM, nk * SF_ATOM, fullS + s);
#pragma unroll
          for (int h = 0; h < 2; ++h)
            tw::bulk_load(sf + (1 + h) * 2 * SF_ATOM, p.sfb0 + ((size_t)(nt * 2 + h) * p.kb + kb0) * SF_ATOM, nk * SF_ATOM, fullS + s);
        }
        __syncwarp();
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 2 || warp == 6) {
    // ------------------------------------------------------------------ producers of repair units
    // Warp 2: the A1 blocks the pair issues (union of both supports); this CTA's own block where it is
    // selected, zeros (a box in a plane beyond the tensor) where only the peer's is. Warp 6: this CTA's
    // 64 rows of every W1 tile and the tile's scales. Bytes complete on the step's stage barrier.
    const bool do_a = warp == 2;
    uint32_t s = 0, ph = 0, sa = 0, pa = 0, sw = 0, pw = 0, it = 0;
    bool ok = true;
    for (int tile = pair; tile < p.tiles && ok; tile += pairs, ++it) {
      const int mbi = 2 * (tile / p.tiles_n) + (int)rank;
      const PairTable& tab = table(it);
      ok = tw::mbar_wait_all(tabFull + it % C::TAB_SLOTS, (it / C::TAB_SLOTS) & 1, abort_flag);
      uint32_t ubits = 0, obits = 0, wbits[2] = {0, 0};
      for (int st = 0; st < steps && ok; ++st) {
        const int kb0 = 2 * st;
        if ((kb0 & 31) == 0) {
          ubits = tab.a_union[kb0 >> 5]; obits = tab.a_own[kb0 >> 5];
          wbits[0] = tab.w1bits[0][kb0 >> 5]; wbits[1] = tab.w1bits[1][kb0 >> 5];
        }
        uint32_t mine = 0, bytes = 0;                            // bit 2j + h: unit of block j (half h for W1)
        if (do_a) {
          mine = (ubits & 1u) | ((ubits & 2u) << 1);
          bytes = __popc(ubits & 3u) * UNIT_A + __popc(obits & 3u) * SF_ATOM;
        } else {
          mine = (wbits[0] & 1u) | ((wbits[0] & 2u) << 1) | ((wbits[1] & 1u) << 1) | ((wbits[1] & 2u) << 2);
          bytes = __popc(mine) * (UNIT_W + SF_ATOM);
        }
        ok = tw::mbar_wait_all(emptyS + s, ph ^ 1, abort_flag);    // the stage barrier is in its next phase
        if (!ok) break;
        if (tw::elect_one()) {
          if (mine) tw::mbar_expect_tx(fullS + s, bytes);
          else tw::mbar_arrive(fullS + s);
        }
        __syncwarp();
#pragma unroll 1
        while (mine && ok) {
          const uint32_t u = __ffs(mine) - 1;
          mine &= mine - 1;
          const int j = (int)(u >> 1), kb = kb0 + j;
          if (do_a) {
            const bool own = (obits >> j) & 1u;
            ok = tw::mbar_wait_all(emptyA1 + sa, pa ^ 1, abort_flag);
            if (!ok) break;
            if (tw::elect_one()) {
              tw::tma_load_3d(smem + C::OFF_A1 + sa * UNIT_A, &tm_a1, kb * 64, mbi * 128, own ? 1 : 2, fullS + s);
              if (own) tw::bulk_load(smem + C::OFF_SFA1 + sa * SF_ATOM, p.sfa1 + ((size_t)mbi * p.kb + kb) * SF_ATOM, SF_ATOM, fullS + s);
            }
            __syncwarp();
            if (++sa == C::A1_SLOTS) { sa = 0; pa ^= 1; }
          } else {
            const int loc = tab.w1loc[u & 1u][kb];
            ok = tw::mbar_wait_all(emptyW1 + sw, pw ^ 1, abort_flag);
            if (!ok) break;
            if (tw::elect_one()) {
              tw::tma_load_2d(smem + C::OFF_W1 + sw * UNIT_W, &tm_w1, 0, loc * 128 + (int)rank * 64, fullS + s);
              tw::bulk_load(smem + C::OFF_SFW1 + sw * SF_ATOM, p.sfbw + (size_t)loc * SF_ATOM, SF_ATOM, fullS + s);
            }
            __syncwarp();
            if (++sw == C::W1_SLOTS) { sw = 0; pw ^= 1; }
          }
        }
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
        ubits >>= 2; obits >>= 2; wbits[0] >>= 2; wbits[1] >>= 2;
      }
      if (tw::elect_one()) tw::mbar_arrive(tabEmpty + it % C::TAB_SLOTS);
      __syncwarp();
    }
  } else if (warp == 1 && rank != 0) {
    // ------------------------------------------------------------------ peer: relay of the stage barrier
    uint32_t s = 0, ph = 0, it = 0;
    bool ok = true;
    for (int tile = pair; tile < p.tiles && ok; tile += pairs, ++it) {
      ok = tw::mbar_wait_all(tabFull + it % C::TAB_SLOTS, (it / C::TAB_SLOTS) & 1, abort_flag);
      for (int st = 0; st < steps && ok; ++st) {
        ok = tw::mbar_wait_all(fullS + s, ph, abort_flag);
        if (!ok) break;
        if (tw::elect_one()) mbar_arrive_cluster(fullS + s, 0);
        __syncwarp();
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
      }
      if (tw::elect_one()) tw::mbar_arrive(tabEmpty + it % C::TAB_SLOTS);
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ leader: MMA issuer of the pair
    bool ok = true;
    constexpr uint32_t IDESC_256 = tw::make_idesc_nvf4(256, 256);
    constexpr uint32_t IDESC_128 = tw::make_idesc_nvf4(256, 128);
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
    uint32_t s = 0, ph = 0, sa = 0, sw = 0, it = 0, tsl = 0, tph = 0;
    bool ready = tw::mbar_test_wait(fullS, 0);
    for (int tile = pair; tile < p.tiles && ok; tile += pairs, ++it) {
      const PairTable& tab = *reinterpret_cast<const PairTable*>(smem + C::OFF_TAB + tsl * C::TAB_BYTES);
      ok = tw::mbar_wait_all(tabFull + tsl, tph, abort_flag);
      // both epilogues of the previous tile have read the columns this accumulator shares with theirs
      // (their tcgen05.ld have completed before they arrive)
      if (ok && it > 0) ok = tw::mbar_wait_all(sharedFree, (it - 1) & 1, abort_flag);
      const uint32_t acc = tmem + (it & 1) * C::ACC_STRIDE;
      uint32_t abits = 0, wbits[2] = {0, 0};
      for (int st = 0; st < steps && ok; ++st) {
        const int kb0 = 2 * st;
        const int nq = p.kb - kb0 >= 2 ? 4 : 2;
        if ((kb0 & 31) == 0) {
          abits = tab.a_union[kb0 >> 5];
          wbits[0] = tab.w1bits[0][kb0 >> 5]; wbits[1] = tab.w1bits[1][kb0 >> 5];
        }
        // units of this step in issue order: bit 3j = A1 of block j, bit 3j + 1 + h = W1 tile (block j, half h)
        const uint32_t units = (abits & 1u) | ((abits & 2u) << 2) | ((wbits[0] & 1u) << 1) | ((wbits[0] & 2u) << 3) |
                               ((wbits[1] & 1u) << 2) | ((wbits[1] & 2u) << 4);
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
              pair_copy_scales(t_sfa0 + 4 * q, DSF | (sf_lo + q * 32));
              pair_copy_scales(t_sfb0 + 8 * q, DSF | (sf_lo + 128 + q * 32));
              pair_copy_scales(t_sfb0 + 8 * q + 4, DSF | (sf_lo + 256 + q * 32));
            }
          }
#pragma unroll
          for (int q = 0; q < 4; ++q)                              // A0 W0
            if (q < nq)
              pair_mma_nvf4(acc, D128 | (a0_lo + 2 * q), D128 | (w0_lo + 2 * q), IDESC_256, t_sfa0 + 4 * q, t_sfb0 + 8 * q, (st | q) != 0);
          uint32_t todo = units, la = sa, lw = sw, a1_lo = 0;
#pragma unroll 1
          while (todo) {
            const uint32_t u = __ffs(todo) - 1;
            todo &= todo - 1;
            const uint32_t j = u >= 3 ? 1u : 0u, t = u - 3 * j;
            if (t == 0) {                                          // A1 block j (union) against the resident W0 stage
              a1_lo = a1_base + la * (UNIT_A >> 4);
              const uint32_t usf = sfa1_base + la * (SF_ATOM >> 4);
              const uint32_t b_lo = w0_lo + 4 * j, sfb = t_sfb0 + 16 * j;
              pair_copy_scales(t_sfa1, DSF | usf);
              pair_copy_scales(t_sfa1 + 4, DSF | (usf + 32));
              pair_mma_nvf4(acc, D64 | a1_lo, D128 | b_lo, IDESC_256, t_sfa1, sfb, 1u);
              pair_mma_nvf4(acc, D64 | (a1_lo + 2), D128 | (b_lo + 2), IDESC_256, t_sfa1 + 4, sfb + 8, 1u);
              if (!p.cross) pair_commit(emptyA1 + la);
              if (++la == C::A1_SLOTS) la = 0;
            } else {                                               // W1 tile (block j, half t - 1) against A0
              const uint32_t w1_lo = w1_base + lw * (UNIT_W >> 4), usf = sfw1_base + lw * (SF_ATOM >> 4);
              const uint32_t a_lo = a0_lo + 4 * j, sfa = t_sfa0 + 8 * j, d = acc + (t - 1) * 128;
              pair_copy_scales(t_sfw1, DSF | usf);
              pair_copy_scales(t_sfw1 + 4, DSF | (usf + 32));
              pair_mma_nvf4(d, D128 | a_lo, D64 | w1_lo, IDESC_128, sfa, t_sfw1, 1u);
              pair_mma_nvf4(d, D128 | (a_lo + 2), D64 | (w1_lo + 2), IDESC_128, sfa + 4, t_sfw1 + 4, 1u);
              if (p.cross && ((units >> (3 * j)) & 1u)) {
                pair_mma_nvf4(d, D64 | a1_lo, D64 | w1_lo, IDESC_128, t_sfa1, t_sfw1, 1u);
                pair_mma_nvf4(d, D64 | (a1_lo + 2), D64 | (w1_lo + 2), IDESC_128, t_sfa1 + 4, t_sfw1 + 4, 1u);
              }
              pair_commit(emptyW1 + lw);
              if (++lw == C::W1_SLOTS) lw = 0;
            }
          }
          if (p.cross && (units & 9u)) {                           // a cross term may have read them last
            pair_commit(emptyA1 + sa);
            if ((units & 9u) == 9u) pair_commit(emptyA1 + (sa + 1 == C::A1_SLOTS ? 0 : sa + 1));
          }
          pair_commit(emptyS + s);
        }
        __syncwarp();
        sa = (sa + __popc(units & 9u)) % C::A1_SLOTS;
        sw = (sw + __popc(units & 54u)) % C::W1_SLOTS;
        if (++s == C::STAGES) { s = 0; ph ^= 1; }
        abits >>= 2; wbits[0] >>= 2; wbits[1] >>= 2;
      }
      if (tw::elect_one()) {
        if (ok) pair_commit(accFull + (it & 1));
        tw::mbar_arrive(tabEmpty + tsl);
      }
      __syncwarp();
      if (++tsl == C::TAB_SLOTS) { tsl = 0; tph ^= 1; }
    }
  } else if (warp >= C::FIRST_EPI_WARP) {
    // ------------------------------------------------------------------ epilogue of this CTA's 128 rows
    const int quad = warp & 3;
    const int group = (warp - C::FIRST_EPI_WARP) >> 2;      // column group: 128 of the 256 columns
    const float alpha = __ldg(p.alpha);
    uint32_t it = 0;
    for (int tile = pair; tile < p.tiles; tile += pairs, ++it) {
      const int mbi = 2 * (tile / p.tiles_n) + (int)rank, nt = tile % p.tiles_n;
      const uint32_t a = it & 1;
      if (!tw::mbar_wait_warp(accFull + a, (it >> 1) & 1, abort_flag)) break;
      tw::tc_fence_after();
      const uint32_t t_base = tmem + ((uint32_t)(quad * 32) << 16) + a * C::ACC_STRIDE + group * 128;
      const int row = mbi * 128 + quad * 32 + lane;
      const int col = nt * 256 + group * 128;
      __nv_bfloat16* dst = p.out + (size_t)row * p.n + col;
      const bool store = row < p.m;
      // accumulator 0 shares its last 64 columns with accumulator 1's first 64: those are read first and the
      // leader's MMA issuer is told before they are converted and stored
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int round = a == 0 ? 1 - i : i;
        uint32_t r[2][32];
        tw::tmem_load_32x32(t_base + round * 64, r[0]);
        tw::tmem_load_32x32(t_base + round * 64 + 32, r[1]);
        tw::tmem_load_wait();
        if (i == 0) {
          tw::tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(sharedFree, 0);
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
  cluster_sync_all();                            // no CTA leaves while its peer may still signal it
  if (warp == 1) { tw::tc_fence_after(); pair_tmem_dealloc(*tmem_slot, C::TM_COLS); }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn pair_encode_fn() {
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

bool pair_map(CUtensorMap* map, int rank, const void* base, const cuuint64_t* dims, const cuuint64_t* strides,
              const cuuint32_t* box, CUtensorMapSwizzle swz) {
  cuuint32_t ones[3] = {1, 1, 1};
  return pair_encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box,
                          ones, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

// Called by tw_fused (tw_fused.cu) after argument validation, for n % 256 == 0 and one A support per row block.
int tw_fused_pair_launch(int m, int n, int k, const void* a_codes, const void* w_codes, const void* sfa, const void* sfb,
                         void* out, const float* alpha, void* workspace, cudaStream_t stream, const TwRepairIO* io,
                         int sms, int dev) {
  using C = PairCfg;
  if (!pair_encode_fn()) return TW_ERR_DRIVER;
  CUtensorMap tm_a0, tm_a1, tm_w0, tm_w1;
  const int planes = io->na > 0 ? 2 : 1;
  {
    cuuint64_t dims[3] = {(cuuint64_t)k / 2, (cuuint64_t)io->mp, (cuuint64_t)planes};
    cuuint64_t strides[2] = {(cuuint64_t)k / 2, (cuuint64_t)io->mp * (k / 2)};
    cuuint32_t box0[3] = {128, 128, 1}, box1[3] = {64, 128, 1};
    if (!pair_map(&tm_a0, 3, a_codes, dims, strides, box0, CU_TENSOR_MAP_SWIZZLE_128B)) return TW_ERR_TENSOR_MAP;
    if (!pair_map(&tm_a1, 3, a_codes, dims, strides, box1, CU_TENSOR_MAP_SWIZZLE_64B)) return TW_ERR_TENSOR_MAP;
  }
  {
    cuuint64_t dims[2] = {(cuuint64_t)k / 2, (cuuint64_t)n};
    cuuint64_t strides[1] = {(cuuint64_t)k / 2};
    cuuint32_t box[2] = {128, 128};
    if (!pair_map(&tm_w0, 2, w_codes, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B)) return TW_ERR_TENSOR_MAP;
  }
  {
    const bool has = io->hasw != 0;
    cuuint64_t dims[2] = {64, (cuuint64_t)(has ? (size_t)io->bank_blocks * 128 : 128)};
    cuuint64_t strides[1] = {64};
    cuuint32_t box[2] = {64, 64};
    if (!pair_map(&tm_w1, 2, has ? (const void*)io->wr : w_codes, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_64B))
      return TW_ERR_TENSOR_MAP;
  }
  PairParams p{};
  p.sfa0 = static_cast<const uint8_t*>(sfa);
  p.sfa1 = io->a1s_swz;
  p.sfb0 = static_cast<const uint8_t*>(sfb);
  p.sfbw = io->wrs_swz;
  p.wi = io->wi; p.off = io->off; p.wloc = io->wloc; p.mask = io->mask;
  p.alpha = alpha;
  p.bias = static_cast<const __nv_bfloat16*>(io->bias);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = static_cast<int*>(workspace);
  p.m = m; p.n = n; p.k = k; p.na = io->na; p.hasw = io->hasw; p.cross = io->cross;
  p.shared = io->shared; p.dense = io->dense;
  p.kb = k / 128; p.nb = n / 128; p.mb = (m + 127) / 128;
  p.tiles_n = n / 256;
  p.tiles = ((p.mb + 1) / 2) * p.tiles_n;
  static std::atomic<bool> configured[64];       // per-device attributes of the function
  if (!configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(fused_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
      return TW_ERR_LAUNCH;
    configured[dev].store(true, std::memory_order_release);
  }
  cudaLaunchConfig_t cfg{};
  cfg.blockDim = dim3(C::THREADS); cfg.dynamicSmemBytes = C::SMEM_BYTES; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  // persistent grid: as many pairs as can be resident at once (queried once per device)
  static std::atomic<int> resident[64];
  int max_pairs = resident[dev].load(std::memory_order_acquire);
  if (max_pairs == 0) {
    cfg.gridDim = dim3(sms);
    if (cudaOccupancyMaxActiveClusters(&max_pairs, fused_pair_kernel, &cfg) != cudaSuccess || max_pairs <= 0) max_pairs = sms / 2;
    resident[dev].store(max_pairs, std::memory_order_release);
  }
  const int pairs = p.tiles < max_pairs ? p.tiles : max_pairs;
  cfg.gridDim = dim3(2 * pairs);
  return cudaLaunchKernelEx(&cfg, fused_pair_kernel, tm_a0, tm_a1, tm_w0, tm_w1, p) == cudaSuccess ? TW_OK : TW_ERR_LAUNCH;
}
