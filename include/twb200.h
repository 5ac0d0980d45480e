/* C ABI of libtwb200: B200 (sm_100a) kernels for ThunderWorld's selective-FP4-repair path.
 *
 * Conventions (same as the reference's CUTLASS bridge,
 * packages/fp4-repair/src/thunderworld_fp4/cutlass/fused.cu:65-88 and cutlass/backend.py:48-71):
 *   - every pointer is a device pointer owned by the caller unless it is an argument struct;
 *   - the library allocates nothing, keeps no state between calls and never synchronises;
 *   - `stream` is a raw cudaStream_t; every call is legal inside CUDA Graph stream capture;
 *   - the return value is 0 on success, otherwise a code that tw_status() turns into text;
 *   - no C++ exception crosses the boundary.
 *
 * NVFP4 operand format (reference: thunderworld_fp4/cosmos/calibration.py:24-54):
 *   codes   uint8 [planes, rows, K/2]   two E2M1 values per byte, even k in the low nibble
 *   scales  uint8 [planes, rows, K/16]  E4M3 bytes, one per 16 consecutive k, row-major
 *   factor  float                        one per tensor (max|x| / 2688, 1.0 for an all-zero tensor)
 * plane 0 = base, plane 1 = residual of the same tensor under the same factor.
 * "atom layout" of a scale matrix [rows, K/16] (rows padded to a multiple of 128):
 *   offset(r, c) = (r/128)*128*(K/16) + (c/4)*512 + (r%32)*16 + ((r%128)/32)*4 + c%4
 * (reference: cutlass/packing.py:24-25), the layout block-scaled tensor-core MMAs read.
 */
#ifndef TWB200_H
#define TWB200_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- status ------------------------------------------------------------------------------ */
/* Replaces tw_status of cutlass/fused.cu:86-88. Never returns NULL. */
const char* tw_status(int status);
/* Library ABI version (bumped when a struct below changes). */
int tw_abi_version(void);
/* Self-test of the bounded device-side waits (no counterpart in the reference): launches one small CTA whose
 * warps wait on a barrier that nothing signals; after `limit_cycles` SM cycles they give up and the first word of
 * `workspace` becomes the "bounded device-side wait ran out" status. The GPU is neither hung nor faulted. */
int tw_selftest_bounded_wait(void* workspace, long long limit_cycles, void* stream);

/* ---- activation quantizer ------------------------------------------------------------------
 * One call replaces the reference's launch chain scaled_amax -> finish_amax -> pack_activation
 * (thunderworld_fp4/linear.py:13-25, _linear_kernels.py:8-56), its calibrated twin
 * (_calibrated.py:60-71), the current-residual selector base_summary -> choose -> residual_only
 * (_sparse_pack.py:77-93) and the direct atom-layout scale producer (cutlass/packing.py:85-109).
 */
typedef struct TwQuantizeArgs {
  const void* x;            /* bf16 [m, k], contiguous */
  const float* prescale;    /* [k] multiplied in before bf16 rounding, or NULL for ones */
  const float* sensitivity; /* [k], selector weights (repair == 3), else NULL */
  float* factor;            /* out: tensor factor; in when factor_given != 0 */
  const float* wg;          /* optional: weight global scale, to emit alpha = factor * wg */
  float* alpha;             /* optional out (needs wg) */
  uint8_t* codes;           /* out [planes, mp, k/2] */
  uint8_t* scales;          /* out [planes, mp, k/16] row-major E4M3 bytes */
  uint8_t* scales_swz;      /* optional out [planes, ceil(m/128)*128, k/16] atom layout */
  uint8_t* mask;            /* bool bytes [ceil(m/128), k/128]: in for repair == 2, out for repair == 3 */
  void* workspace;          /* tw_quantize_workspace(m, k) bytes of scratch */
  int m, k, mp;             /* mp: rows per plane of codes / scales, a multiple of 16 >= m (ceil(m/16)*16 when the planes
                               hold this call's rows only; larger when they are a shard of a wider gathered tensor) */
  int repair;               /* 0 base plane only; 1 residual everywhere; 2 residual where mask is set,
                               zero codes and scales elsewhere; 3 residual everywhere and mask := the
                               top-`na` K128 blocks per M128 row block ranked by residual energy */
  int na;                   /* quota for repair == 3 (0 < na < k/128) */
  int factor_given;         /* nonzero: read *factor instead of reducing max|x| */
  float base, res, gain;    /* scale multipliers of the calibrated packer; 1,1,1 = plain */
  float energy;             /* < 1: energy-prefix stop of the selector; 1 = off */
  int swz_rows;             /* rows per plane of scales_swz; 0 = ceil(m/128)*128, else a multiple of 128 not below that */
} TwQuantizeArgs;
size_t tw_quantize_workspace(int m, int k);
int tw_quantize(const TwQuantizeArgs* args, void* stream);

/* tw_quantize without caller-provided scratch. No counterpart in the reference: it serves hosts that may
 * not allocate device memory where they quantize (a plugin inside another framework's memory plan, a loop
 * that forbids allocation after start-up). `args->workspace` is ignored; the scratch is a fixed array inside
 * the library, one per GPU, held until the process exits. Limit: ceil(m/128) * (k/128) <=
 * tw_quantize_static_max_tiles() (16384), larger problems return the "size exceeds the stated maximum" status.
 * The first call on a device looks the array's address up and should come before any stream capture. All
 * calls on a device share the array: calls that overlap on the GPU race. Allocates nothing. */
int tw_quantize_static(const TwQuantizeArgs* args, void* stream);
int tw_quantize_static_max_tiles(void);

/* Sampled-energy rank of every K128 block within its M128 row block: rank int32 [ceil(m/128), k/128], 0 = largest
 * (eight rows x eight columns of bf16(x * prescale) per 128x128 block; the lower index wins ties). prescale may be
 * NULL. Replaces activation_rank of thunderworld_fp4/_linear_kernels.py:23-34 (one launch, no host sync). */
int tw_activation_rank(const void* x_bf16, const float* prescale, int m, int k, int32_t* rank, void* stream);

/* Row-major E4M3 scale bytes [rows, cols] -> atom layout [ceil(rows/128)*128, cols], padding zeroed.
 * Replaces thunderworld_fp4/cutlass/layout.py:7-25 (swizzle). cols % 4 == 0. */
int tw_swizzle_scales(const uint8_t* src, int rows, int cols, uint8_t* dst, void* stream);

/* ---- fused repair GEMM ---------------------------------------------------------------------
 * out[m, n] (bf16) = alpha * ( A0 W0^T + sum_{kb in support(mb)} A1[kb] W0[kb]^T
 *                            + sum_{(nb,kb) in tiles} A0[kb] W1[nb,kb]^T
 *                            [+ A1[kb] W1[nb,kb]^T where both are selected, if cross] )
 * with one fp32 accumulator per output element and one bf16 rounding.
 * Same entry point, argument order and meaning as tw_fused of cutlass/fused.cu:78-85 and its
 * tcgen05 twin tools/thor_handoff/cutlass_sm110_fused.cu:57-77. The struct below starts with the
 * reference's RepairIO (cutlass/repair_collective.cuh:5-10, bank_blocks from
 * tools/thor_handoff/sm110_repair_collective.cuh:6-11) and appends the atom-layout scale pointers
 * of the residual operands, which this implementation requires whenever those terms are issued.
 */
typedef struct TwRepairIO {
  const uint8_t *ac, *as, *wc, *ws, *wr, *wrs; /* activation codes/scales (planes), W0 codes/scales,
                                                  W1 bank codes [slots,128,64] / scales [slots,128,8] */
  const int32_t *wi, *off, *wloc;              /* CSR over N128 blocks: k-block per slot, row offsets
                                                  [n/128+1], bank position per slot */
  const uint8_t* mask;                         /* bool [ceil(m/128), k/128], read at run time */
  int32_t m, mp, n, k, na, hasw, cross, shared, dense, bank_blocks; /* mp: rows per plane of ac / as, a multiple of 16 >= m */
  /* extensions */
  const uint8_t* a1s_swz;  /* residual-plane activation scales, atom layout [ceil(m/128)*128, k/16] */
  const uint8_t* wrs_swz;  /* W1 bank scales, atom layout per tile: [slots][1024] */
  const void* bias;        /* optional bf16 [n]: out = bf16(alpha * acc + bias), one rounding, as the reference's
                              FP4Linear kernel does (thunderworld_fp4/_linear_kernels.py:79-81) */
  int32_t mask_per_n;      /* nonzero: mask is bool [ceil(m/128), n/128, k/128], one A support per output
                              block (explicit masks of FP4Linear, thunderworld_fp4/linear.py:115-119) */
  int32_t kernel;          /* 0: the library chooses (today: the single-CTA kernel); 1: single-CTA kernel; 2: CTA-pair kernel (cta_group::2;
                              needs n % 256 == 0, m > 128 and no mask_per_n). Both give the same bits. */
  int32_t activation;      /* 0: none. TW_ACT_GELU_TANH: out = bf16(gelu_tanh(bf16(alpha * acc + bias))), bit for bit what
                              tw_activate produces from this call's plain output (the FFN-up projection followed by
                              activate_with_factor, thunderworld_fp4/_fusion.py:26-34, in one pass; single-CTA kernel only) */
  float* stats;            /* with an activation, optional: {max|out| / 2688 (1 for an all-zero out), max|out|} over the m x n
                              output, written by the last CTA to finish */
  uint32_t* stats_scratch; /* two zeroed words (required with stats); left zeroed */
} TwRepairIO;
/* Limits: n % 128 == 0, k % 128 == 0, k <= 24576 (else the "size exceeds the stated maximum" status).
 * Bytes of caller-owned workspace (holds the device status word; zero it once). */
size_t tw_workspace(int m, int n, int k);
int tw_fused(int m, int n, int k, const void* a_codes, const void* w_codes, const void* sfa_swz,
             const void* sfb_swz, void* out_bf16, const float* alpha_dev, void* workspace, void* stream,
             const TwRepairIO* io);
/* N extent of the output tile the kernel uses for this n (256, or 128 when n is an odd multiple of
 * 128). Pure host function. */
int tw_fused_tile_n(int n);

/* ---- streaming FP4 attention -----------------------------------------------------------------
 * Three calls replace the reference's attention launch chain (thunderworld_fp4/runtime.py:32-108):
 *   tw_pack_rows     pack_qk / pack_v        (_kernels.py:12-47): per-row factor max/1536, base + residual
 *   tw_select_tiles  select_tiles[_head]     (_kernels.py:169-215): per-head quota of repaired key tiles
 *   tw_attention     streaming_attention     (_kernels.py:51-124); no split/combine pass is needed
 * Packed layouts: codes [planes, heads*rows_padded, 64], scales [planes, heads*rows_padded, 8] (row-major),
 * scales_swz [planes, heads, ceil(rows_padded/128), 1024] (atom layout), factors [heads*rows_padded].
 * Q and K rows are (head, token); V rows are (kv head, key tile, channel) with the tile's 128 tokens as
 * columns (rows_padded = key tiles * 128). */
typedef struct TwPackRowsArgs {
  const void* x;                 /* bf16, element (token, head, d) at x[token*stride_row + head*stride_head + d] */
  uint8_t *codes, *scales, *scales_swz;
  float* factors;
  float* energy;                 /* V only, optional: [heads, key tiles, 8] = sum x^2 / 16384 per 16 channels */
  long long stride_row, stride_head;
  int rows, heads, rows_padded;  /* tokens, heads, padded rows per head (16-multiple; 128-multiple for V) */
  int repair;                    /* also emit the residual plane */
  int transpose_v;               /* 0: Q/K packing, 1: V packing */
  int need_energy;
} TwPackRowsArgs;
int tw_pack_rows(const TwPackRowsArgs* args, void* stream);

typedef struct TwSelectArgs {
  const void *q, *k;             /* bf16 inputs with the strides below */
  const float* energy;           /* from tw_pack_rows on V */
  int32_t *flags, *pvflags;      /* out [hq, ceil(m/128), ceil(n/128)]: `terms` where repaired, else 1 */
  const int32_t *counts, *pvcounts; /* per query head quotas (device) */
  long long q_stride_row, q_stride_head, k_stride_row, k_stride_head;
  int m, n, hq, hk, terms, pv_terms;
} TwSelectArgs;
int tw_select_tiles(const TwSelectArgs* args, void* stream);

typedef struct TwAttentionArgs {
  const uint8_t *qc, *kc, *vc;   /* codes */
  const uint8_t *sfq, *sfk, *sfv;/* atom-layout scales */
  const float *qf, *kf, *vf;     /* factors */
  const int32_t *flags, *pvflags;/* > 1 selects repair of that (head, q block, key tile); may be NULL when full / off */
  void* out;                     /* bf16 [m, hq, 128] */
  void* workspace;               /* tw_attention_workspace bytes; first word = device status */
  int m, n, hq, hk, mp, np;      /* mp = ceil(m/16)*16, np = ceil(n/128)*128 */
  int repair, full, terms;       /* QK: any repair, every tile repaired, 2/3/4 terms */
  int pv_repair, pv_full, pv_terms;
} TwAttentionArgs;
size_t tw_attention_workspace(int m, int n, int hq, int hk);
int tw_attention(const TwAttentionArgs* args, void* stream);

/* ---- pointwise producers with fused tensor factor ------------------------------------------
 * Each writes its bf16 result once and, when `stats` is given, reduces max|y| in the same pass:
 * stats[0] = factor = max|y| / 2688 (1.0 for an all-zero tensor, thunderworld_fp4/_linear_kernels.py:17-19
 * finish_amax), stats[1] = max|y|. The factor feeds tw_quantize with factor_given, which then skips its own
 * reduction pass (the reference's pack_with_factor, thunderworld_fp4/_fusion.py:37-42).
 * `scratch`: 8 bytes of device memory, zeroed once by the caller; every call leaves it zeroed. Calls that
 * share a scratch must not overlap on the GPU. */
enum { TW_ACT_RELU2 = 0, TW_ACT_MUL = 1, TW_ACT_GELU_TANH = 2 };
/* y = bf16(relu(a)^2) | bf16(a * b) | bf16(gelu_tanh(a)); fp32 arithmetic, one rounding. n % 8 == 0.
 * Modes 0 and 1 replace pointwise_amax / activate_with_factor (thunderworld_fp4/_fusion.py:15-34) and are
 * bit-exact against them; mode 2 is the activation of the DiT step's FFN. */
int tw_activate(const void* a, const void* b, void* y, float* stats, void* scratch, long long n, int mode, void* stream);
/* y[r, :] = bf16( x[r, :] * rsqrt(mean(x[r, :]^2) + eps) [* weight] [* (1 + scale[b, :]) + shift[b, :]] ), b = r /
 * rows_per_batch. weight, shift, scale: bf16 or NULL (shift and scale together). Replaces nemotron_norm
 * (thunderworld_fp4/cosmos/norm_fusion.py:23-43) plus the AdaLN modulation that follows it in a DiT block.
 * hidden % 8 == 0, hidden <= 16384. */
int tw_rms_norm(const void* x, const void* weight, const void* shift, const void* scale, void* y, float* stats,
                void* scratch, int rows, int hidden, int rows_per_batch, float eps, void* stream);
/* RMSNorm over the last dimension (128) of a strided bf16 view [tokens, heads, 128] (query / key norm);
 * y is contiguous [tokens, heads, 128]. Strides in elements, multiples of 8. */
int tw_rms_norm_heads(const void* x, void* y, long long tokens, int heads, long long stride_token, long long stride_head,
                      float eps, void* stream);
/* Rotary embedding of 128-wide head rows of a strided bf16 view [tokens, heads, 128], with the reference's rounding
 * sequence (thunderworld_fp4/cosmos/pipeline_tuning.py:42-63, fused_rope): y[d] = bf16(bf16(x[d] cos[d]) + bf16(rot[d]
 * sin[d])), rot[d] = -x[d + 64] (d < 64) or x[d - 64]. cos / sin tables are [table_rows, 128], float32 or bf16, 16-byte aligned; row
 * token % table_rows applies to a token. norm != 0: the head RMSNorm of tw_rms_norm_heads runs first in the same pass
 * (its bf16 result is what gets rotated, as when the two kernels run one after the other). */
int tw_rope_heads(const void* x, void* y, long long tokens, int heads, long long stride_token, long long stride_head,
                  const void* cos_table, const void* sin_table, long long table_rows, int table_is_bf16, int norm,
                  float eps, void* stream);
/* x[r, :] = bf16(x[r, :] + gate[r / rows_per_batch, :] * y[r, :]) in place (gated residual of a DiT block). */
int tw_gate_residual(void* x, const void* gate, const void* y, int rows, int hidden, int rows_per_batch, void* stream);

#ifdef __cplusplus
}
#endif
#endif
