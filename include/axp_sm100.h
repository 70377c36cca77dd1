/*
 * C-ABI launch shim for the sm100 (B200, sm_100a) realizations of iro-cuda-ax's
 * L3 `gemm` and `attention` recipes.
 *
 * The reference library is a compile-time contract library with no launch layer
 * ("does not provide runtime orchestration or a kernel launch framework",
 * README.md:20); its user writes the __global__ kernel and calls the selected
 * realizations' execute() members (examples/sm89_ax_div_example.cu:20-41,68-72).
 * This header is that hand-written kernel layer for sm100, exported so that C,
 * C++ or any FFI can launch it.  Each entry point names the reference interface
 * it stands behind.
 *
 * Conventions (all entry points):
 *   - plain pointers and sizes only; every data pointer is a DEVICE pointer owned
 *     by the caller; nothing is allocated, freed or synchronised on the caller's
 *     behalf; work is enqueued on `stream` (a cudaStream_t passed as void*);
 *   - return value: AXP_OK or a negative AXP_ERR_*; no exception crosses the ABI;
 *     axp_sm100_last_error() returns a thread-local message for the last failure;
 *   - `status_dev` (may be NULL) points to one 32-bit device word, zeroed by the
 *     caller.  A kernel whose bounded wait runs out ORs a non-zero code into it
 *     (bit 31 set) and unwinds without hanging; the caller reads it after
 *     synchronising the stream and treats non-zero as AXP_ERR_TIMEOUT;
 *   - calls on distinct streams may be made from distinct host threads.
 */
#ifndef AXP_SM100_H_
#define AXP_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AXP_OK 0
#define AXP_ERR_BAD_ARG (-1)
#define AXP_ERR_UNSUPPORTED (-2)
#define AXP_ERR_CUDA (-3)
#define AXP_ERR_TIMEOUT (-4)

/* What one realization key resolves to.  The key is fnv1a_64 of the manifest
 * row's `realization_key` string, the same value the reference's generated
 * registry stores (include/axp/l4/graph_registry_index.hpp:149-156) and
 * axp::l4::resolve<>::realization_key exposes (include/axp/l4/resolve.hpp:52). */
typedef struct axp_sm100_caps {
    uint64_t realization_key; /* echo of the queried key                        */
    int32_t op_family;        /* 1 = gemm, 2 = attention, 3 = gemm_fused         */
    int32_t elem_bits;        /* operand element width: 8 (e4m3) or 16 (bf16)   */
    int32_t tile_m, tile_n, tile_k; /* CTA tile                                 */
    int32_t cta_group;        /* CTAs cooperating on one MMA (1 or 2)           */
    int32_t stages;           /* shared-memory pipeline depth                   */
    int32_t smem_bytes;       /* dynamic shared memory per CTA                  */
    int32_t tmem_columns;     /* tensor-memory columns allocated per CTA        */
    int32_t threads;          /* threads per CTA                                */
} axp_sm100_caps;

/* Replaces: kits/sm100 lookup (`axp::kit::sm100::bind<O>`,
 * include/axp/kits/sm100/registry.hpp:10-20, empty upstream).  Returns
 * AXP_ERR_UNSUPPORTED for a key with no sm100 row. */
int axp_sm100_query(uint64_t realization_key, axp_sm100_caps* out);

/* fnv1a_64 of a NUL-terminated string (include/iro_cuda_ax_core.hpp:245-252), so
 * that FFI callers can form realization keys from manifest strings. */
uint64_t axp_sm100_fnv1a64(const char* s);

/* FP8 E4M3 block-scaled GEMM, bf16 output:
 *   C[m,n] = bf16( sum_kb sA[m,kb] * sB[n/128,kb] * sum_{k in kb} A[m,k]*B[n,k] )
 * A [M,K] row-major (lda elements), B [N,K] K-contiguous (ldb) -- the "TN" operand
 * layout of the reference recipe (include/axp/level3/gemm.hpp:1162-1176); fp32
 * accumulate with one partial per K tile (gemm.hpp:1512-1515); sA [M,K/128] and
 * sB [ceil(N/128),K/128] row-major fp32; C [M,N] bf16 (ldc).  Only output columns
 * [n_begin,n_end) are computed (N-sharding); n_begin must be a multiple of 128 and
 * n_end - n_begin a multiple of 8 (every GEMM entry point of this header writes,
 * and reads bias / C input, eight columns at a time; AXP_ERR_BAD_ARG otherwise).
 * Requires K % 128 == 0, lda/ldb % 16 == 0, ldc % 8 == 0, 16-byte aligned bases.
 * Realizes: GemmTilePattern on cap::sm100 (gemm.hpp:2276-2375 dispatch; the
 * ScaleSharedTile hook gemm.hpp:104-116,1379-1382 becomes a scale-and-promote of
 * the fp32 partial). */
int axp_sm100_gemm_fp8_blockscaled(const void* A, const void* B, const float* sA, const float* sB, void* C,
                                   int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb, int64_t ldc,
                                   int64_t n_begin, int64_t n_end, void* stream, uint32_t* status_dev);

/* BF16 GEMM, fp32 accumulate, bf16 output; layouts as above (no scales).
 * Requires K % 8 == 0, lda/ldb/ldc % 8 == 0, n_begin % 8 == 0.
 * Realizes: GemmTilePattern<BF16AccF32Fast,...> on cap::sm100
 * (include/axp/recipes.hpp:13-14, gemm.hpp:1075-2027). */
int axp_sm100_gemm_bf16(const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                        int64_t ldb, int64_t ldc, int64_t n_begin, int64_t n_end, void* stream,
                        uint32_t* status_dev);

#define AXP_ACT_NONE 0
#define AXP_ACT_SILU 1

/* The two GEMMs with the reference's fused bias + activation epilogue on the fp32
 * accumulator: C = bf16( act( acc + bias[n] ) ), bias fp32 [N] (16-byte aligned),
 * act = AXP_ACT_NONE or AXP_ACT_SILU (x * sigmoid(x)).  Other arguments as above.
 * Realizes: GemmTileFusedPattern with epilogue::BiasActivationVec on cap::sm100
 * (include/axp/level3/gemm.hpp:159-219, preset include/axp/l4/preset/gemm.hpp:33-45,
 * SiLU include/axp/realize/l0.hpp:1955-1965). */
int axp_sm100_gemm_bf16_bias_act(const void* A, const void* B, const float* bias, void* C, int64_t M, int64_t N,
                                 int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int64_t n_begin, int64_t n_end,
                                 int act, void* stream, uint32_t* status_dev);
int axp_sm100_gemm_fp8_blockscaled_bias_act(const void* A, const void* B, const float* sA, const float* sB,
                                            const float* bias, void* C, int64_t M, int64_t N, int64_t K, int64_t lda,
                                            int64_t ldb, int64_t ldc, int64_t n_begin, int64_t n_end, int act,
                                            void* stream, uint32_t* status_dev);

/* Linear-combination epilogue: D = bf16( alpha * acc + beta * Cin ), Cin [M,N] bf16 (ldcin), evaluated as the three
 * fp32 operations MulAcc, MulC, Add of the reference (no contraction); D may be Cin (in-place update).
 * Realizes: GemmTileFusedPattern + epilogue::LinearCombinationVec (include/axp/level3/gemm.hpp:187-208, 221-234). */
int axp_sm100_gemm_bf16_lincomb(const void* A, const void* B, const void* Cin, void* D, float alpha, float beta, int64_t M, int64_t N,
                                int64_t K, int64_t lda, int64_t ldb, int64_t ldcin, int64_t ldd, int64_t n_begin, int64_t n_end,
                                void* stream, uint32_t* status_dev);
int axp_sm100_gemm_fp8_blockscaled_lincomb(const void* A, const void* B, const float* sA, const float* sB, const void* Cin, void* D,
                                           float alpha, float beta, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                           int64_t ldcin, int64_t ldd, int64_t n_begin, int64_t n_end, void* stream,
                                           uint32_t* status_dev);

/* Gate / up projection of a gated MLP in one pass:
 *   H[:, n] = bf16( SiLU( X . Wg[n,:] ) * ( X . Wu[n,:] ) ),  fp32 accumulate,
 * X [M,K] (ldx), Wg and Wu [N,K] K-contiguous (ldwg, ldwu), H [M,N] (ldh), all bf16; only columns
 * [n_begin,n_end) are computed.  Requires K, leading dimensions and n_begin to be multiples of 8.
 * The two products never reach memory: a CTA (pair) accumulates gate and up columns of the same
 * 128 outputs side by side in tensor memory and the epilogue combines them.
 * Realizes: GemmTileFusedPattern with a gated activation epilogue (the SiLU preset of
 * include/axp/l4/preset/gemm.hpp:33-45 applied to the Llama MLP gate/up pair). */
int axp_sm100_gemm_bf16_swiglu(const void* X, const void* Wg, const void* Wu, void* H, int64_t M, int64_t N, int64_t K,
                               int64_t ldx, int64_t ldwg, int64_t ldwu, int64_t ldh, int64_t n_begin, int64_t n_end,
                               void* stream, uint32_t* status_dev);

/* The same gate / up pass on E4M3 block-scaled operands: X [M,K] with 1x128 scales sX [M,K/128], Wg and Wu
 * [N,K] with 128x128 scales sWg, sWu [ceil(N/128),K/128]; both products are promoted per 128-wide K block
 * exactly as in axp_sm100_gemm_fp8_blockscaled (acc += (sX*sW) * partial), combined in fp32 and rounded
 * once to bf16.  Requires K % 128 == 0, n_begin % 128 == 0, operand leading dimensions % 16, ldh % 8.
 * Realizes: the block-scaled main loop of include/axp/level3/gemm.hpp:221-234 with the gated activation
 * epilogue of the bf16 entry point above. */
int axp_sm100_gemm_fp8_blockscaled_swiglu(const void* X, const void* Wg, const void* Wu, const float* sX, const float* sWg,
                                          const float* sWu, void* H, int64_t M, int64_t N, int64_t K, int64_t ldx, int64_t ldwg,
                                          int64_t ldwu, int64_t ldh, int64_t n_begin, int64_t n_end, void* stream,
                                          uint32_t* status_dev);

/* The block-scaled GEMM (optionally with the bias / activation epilogue) with a quantising epilogue: instead of bf16 C it
 * leaves Cq [M,N] E4M3 bytes (ldq bytes per row, a multiple of 16) and Cq_scales [M, N/128] fp32, bit for bit what
 * axp_sm100_quantize_rows_e4m3 produces from the bf16 C of axp_sm100_gemm_fp8_blockscaled(_bias_act): an epilogue thread
 * owns one 128-column scale block of its row.  bias may be null (act is then ignored).  Requires N % 128 == 0 and a
 * column range of whole 128-column blocks.  Realizes the reference's CastTile with the fp8_saturate policy
 * (include/axp/protocol/convert/contracts.hpp:31, include/axp/detail/conversion.hpp:83-95) behind the GEMM recipe. */
int axp_sm100_gemm_fp8_blockscaled_quant(const void* A, const void* B, const float* sA, const float* sB, const float* bias, int act,
                                         void* Cq, float* Cq_scales, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                                         int64_t ldq, int64_t n_begin, int64_t n_end, void* stream, uint32_t* status_dev);

/* The same pass with a quantising epilogue: instead of bf16 H it leaves Hq [M,N] E4M3 bytes (leading dimension ldq
 * bytes, a multiple of 16) and Hq_scales [M, N/128] fp32 - the A operand and the 1x128 scales of the next block-scaled
 * GEMM (the MLP's down projection) - bit for bit what axp_sm100_quantize_rows_e4m3 produces from the bf16 H of the
 * entry point above: the value is rounded to bf16 in registers, the block maximum of a row's 128 output columns is
 * formed by the row's two epilogue threads, scale = max / 448, q = e4m3_sat(h * (1 / scale)).  H itself never reaches
 * HBM.  Requires N % 128 == 0 and a column range of whole 128-column blocks; rank-sharded calls write their blocks of
 * Hq_scales.  Realizes: the gated epilogue above followed by the reference's CastTile with the fp8_saturate policy
 * (include/axp/protocol/convert/contracts.hpp:31, include/axp/detail/conversion.hpp:83-95). */
int axp_sm100_gemm_fp8_blockscaled_swiglu_quant(const void* X, const void* Wg, const void* Wu, const float* sX, const float* sWg,
                                                const float* sWu, void* Hq, float* Hq_scales, int64_t M, int64_t N, int64_t K,
                                                int64_t ldx, int64_t ldwg, int64_t ldwu, int64_t ldq, int64_t n_begin, int64_t n_end,
                                                void* stream, uint32_t* status_dev);

/* Flash-attention forward, bf16, per-row online softmax.
 * Q [B,Hq,S,D], K,V [B,Hkv,S,D], O [B,Hq,S,D] bf16 contiguous; LSE [B,Hq,S] fp32
 * (may be NULL).  s = scale * q.k, optional causal mask (key <= query), kv head =
 * h / (Hq/Hkv).  Only flattened heads b*Hq+h in [bh_begin,bh_end) are computed.
 * Requires D == 128 and S % 8 == 0.
 * Realizes: AttentionTilePattern on cap::sm100 (include/axp/level3/attention.hpp:792-846;
 * dataflow include/axp/level3/recipes/attention/process.hpp:1766-1864 with the
 * softmax state taken per query row). */
int axp_sm100_attn_fwd_bf16(const void* Q, const void* K, const void* V, void* O, float* LSE, int64_t B,
                            int64_t Hq, int64_t Hkv, int64_t S, int64_t D, float scale, int causal,
                            int64_t bh_begin, int64_t bh_end, void* stream, uint32_t* status_dev);

/* FP8 (E4M3) flash-attention forward with GQA.  Q,K,V are E4M3 bytes in the
 * layouts above; q_descale [B*Hq], k_descale/v_descale [B*Hkv] fp32;
 * s = scale*dq*dk*(q.k); P is quantised to E4M3 with saturation before P.V
 * (include/axp/detail/conversion.hpp:83-95); O = bf16(dv * P.V / l).
 * Requires D == 128 and S % 16 == 0. */
int axp_sm100_attn_fwd_fp8(const void* Q, const void* K, const void* V, const float* q_descale,
                           const float* k_descale, const float* v_descale, void* O, float* LSE, int64_t B,
                           int64_t Hq, int64_t Hkv, int64_t S, int64_t D, float scale, int causal,
                           int64_t bh_begin, int64_t bh_end, void* stream, uint32_t* status_dev);

/* Producer of the FP8 GEMM's A operand: bf16 X [M,K] (ldx) -> E4M3 Q [M,K] (ldq) and fp32 scales
 * [M, K/128] (contiguous), one scale per row per 128-wide K block:
 *   scale = max|x| / 448 over the block (1 for an all-zero block),  q = e4m3_sat( x * (1/scale) ).
 * Q and scales are exactly the A / sA arguments of axp_sm100_gemm_fp8_blockscaled.
 * Requires K % 128 == 0, ldx/ldq % 8 == 0, X 16-byte and Q 8-byte aligned.
 * Stands behind: CastTile with the fp8_saturate policy (include/axp/protocol/convert/contracts.hpp:31,
 * include/axp/detail/conversion.hpp:83-95). */
int axp_sm100_quantize_rows_e4m3(const void* X, void* Q, float* scales, int64_t M, int64_t K, int64_t ldx, int64_t ldq,
                                 void* stream);

/* RMSNorm fused with the quantiser: y = (x * inv_rms) * w with inv_rms = 1 / sqrt(mean(x^2) + eps), W [K] bf16, then
 * the 1x128 quantisation of axp_sm100_quantize_rows_e4m3 applied to y (the normalised row is never written);
 * K a multiple of 128 and at most 16384.  Every arithmetic step is one IEEE fp32 operation in a fixed order, so the
 * result is bit-exact against the CPU restatement.
 * Realizes: the RMSNorm fragment recipe (include/axp/level3/domain/norm.hpp:610-634, inv_rms norm.hpp:436-445) feeding
 * CastTile / fp8_saturate (include/axp/detail/conversion.hpp:83-95). */
int axp_sm100_rmsnorm_quantize_rows_e4m3(const void* X, const void* W, float eps, void* Q, float* scales, int64_t M, int64_t K,
                                         int64_t ldx, int64_t ldq, void* stream);

/* Split-KV attention (decode, chunked prefill, few heads): Q [B,Hq,Sq,D], K / V [B,Hkv,Skv,D], O [B,Hq,Sq,D] bf16,
 * LSE [B,Hq,Sq] f32 or NULL.  Under the causal mask query i sees keys 0 .. i + (Skv - Sq) (Sq <= Skv required).  The keys
 * are cut into num_splits shares of whole KV tiles; every share is an independent pass of the forward kernel (grid z)
 * that leaves its unnormalised fp32 accumulator and (m, l) per row in `scratch`; a second kernel combines the shares:
 *   m = max_z m_z,  O = sum_z e^(m_z - m) O_z / sum_z e^(m_z - m) l_z.
 * Calls with at most 16 query rows per KV head (the query heads of a GQA group counted together) run a decode kernel
 * instead, which puts the 128 keys of a KV tile on the tensor-memory lanes and the query rows on 16 accumulator columns
 * (S^T = K.Q^T, O^T = V^T.P^T); partial results, scratch size and combine are the same, and with num_splits = 1 it
 * writes O and LSE itself.
 * `scratch` is caller-owned device memory, 256-byte aligned, of at least
 * axp_sm100_attn_splitkv_scratch_bytes(bh_end - bh_begin, Sq, num_splits) bytes (0 for num_splits = 1); the library
 * allocates nothing.  Realizes the softmax state combine of the reference recipe across KV ranges
 * (include/axp/level3/recipes/attention/process.hpp:154-159, 853-860). */
int64_t axp_sm100_attn_splitkv_scratch_bytes(int64_t heads, int64_t Sq, int64_t num_splits);
int axp_sm100_attn_fwd_bf16_splitkv(const void* Q, const void* K, const void* V, void* O, float* LSE, int64_t B, int64_t Hq,
                                    int64_t Hkv, int64_t Sq, int64_t Skv, int64_t D, float scale, int causal,
                                    int64_t num_splits, void* scratch, int64_t scratch_bytes, int64_t bh_begin,
                                    int64_t bh_end, void* stream, uint32_t* status_dev);
/* The same on an E4M3 KV cache: Q, K, V E4M3 with one fp32 descale per (batch, head) as in axp_sm100_attn_fwd_fp8
 * (q_descale [B*Hq], k_descale and v_descale [B*Hkv]); Skv % 16 == 0.  With few queries per head (2 * Sq <= 128) the
 * query heads of a GQA group share one pass over their K / V, each row with its own head's Q descale.
 * Realizes: the FP8 attention recipe (include/axp/level3/recipes/attention/fp8_policy.hpp:21-40) with the same combine. */
int axp_sm100_attn_fwd_fp8_splitkv(const void* Q, const void* K, const void* V, const float* q_descale, const float* k_descale,
                                   const float* v_descale, void* O, float* LSE, int64_t B, int64_t Hq, int64_t Hkv, int64_t Sq,
                                   int64_t Skv, int64_t D, float scale, int causal, int64_t num_splits, void* scratch,
                                   int64_t scratch_bytes, int64_t bh_begin, int64_t bh_end, void* stream, uint32_t* status_dev);

/* Attention over a KV shard (context / sequence parallelism: every GPU holds a slice of the keys): the forward pass
 * over local keys [kv_pos0, kv_pos0 + Skv_local) of a sequence of Skv_total keys that leaves, instead of O and LSE, one
 * partial result: [rows][128] fp32 unnormalised accumulators followed by [rows] (m, l) pairs, rows = (bh_end - bh_begin)
 * * Sq, axp_sm100_attn_partial_bytes(heads, Sq) bytes, 256-byte aligned, caller-owned.  Under the causal mask query i
 * sees global key positions <= i + (Skv_total - Sq).  axp_sm100_attn_combine_partials merges num_shares such results
 * (share z at partials + z * share_stride_bytes; e.g. the all-gathered results of all ranks) into O [rows,128] bf16 and
 * LSE [rows]: the softmax state combine of the reference recipe (process.hpp:107-164) across GPUs.  The exchange
 * itself (an all-gather of the partial results) is the caller's; `shard.attn_kv_sharded` does it with torch.distributed. */
int64_t axp_sm100_attn_partial_bytes(int64_t heads, int64_t Sq);
int axp_sm100_attn_fwd_bf16_kvshard(const void* Q, const void* K, const void* V, void* partial, int64_t partial_bytes, int64_t B,
                                    int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv_local, int64_t kv_pos0, int64_t Skv_total,
                                    int64_t D, float scale, int causal, int64_t bh_begin, int64_t bh_end, void* stream,
                                    uint32_t* status_dev);
/* The same pass on E4M3 operands (Q, K, V bytes and per-head descales as for axp_sm100_attn_fwd_fp8): the partial result has
 * the same layout and merges with axp_sm100_attn_combine_partials.  As in axp_sm100_attn_fwd_fp8_splitkv, every shard
 * rounds its softmax weights to E4M3 against its own running maximum. */
int axp_sm100_attn_fwd_fp8_kvshard(const void* Q, const void* K, const void* V, const float* q_descale, const float* k_descale,
                                   const float* v_descale, void* partial, int64_t partial_bytes, int64_t B, int64_t Hq, int64_t Hkv,
                                   int64_t Sq, int64_t Skv_local, int64_t kv_pos0, int64_t Skv_total, int64_t D, float scale,
                                   int causal, int64_t bh_begin, int64_t bh_end, void* stream, uint32_t* status_dev);
int axp_sm100_attn_combine_partials(const void* partials, int64_t num_shares, int64_t share_stride_bytes, void* O, float* LSE,
                                    int64_t rows, void* stream);

/* The same split-KV attention with its scratch memory inside the library: a file-scope, 256-byte aligned device array
 * of axp_sm100_attn_splitkv_static_scratch_bytes() = 16 MiB, whose address is looked up once per device.  The call
 * allocates and frees nothing; it returns AXP_ERR_BAD_ARG when num_splits * (bh_end - bh_begin) * Sq rows of
 * (128 * 4 + 8) bytes do not fit.  All calls on a device share the array, so they must not overlap in time.
 * No counterpart in the reference (its recipes are compile-time and own no memory). */
int64_t axp_sm100_attn_splitkv_static_scratch_bytes(void);
int axp_sm100_attn_fwd_bf16_splitkv_static(const void* Q, const void* K, const void* V, void* O, float* LSE, int64_t B,
                                           int64_t Hq, int64_t Hkv, int64_t Sq, int64_t Skv, int64_t D, float scale,
                                           int causal, int64_t num_splits, int64_t bh_begin, int64_t bh_end, void* stream,
                                           uint32_t* status_dev);

/* Causal mask bits and whole-tile skip predicate for one (tile_m x tile_n) tile,
 * computed on the device by the same code the attention kernels use: bit
 * (row*tile_n+col) of mask_dev is set when k_base+col <= q_base+row; *skip_dev = 1
 * when k_base > q_base+tile_m-1.  Mirrors CausalMaskPred
 * (include/axp/realize/l0.hpp:2563-2623).  mask_dev holds
 * ceil(tile_m*tile_n/64) 64-bit words. */
int axp_sm100_causal_mask_tile(int64_t q_base, int64_t k_base, int32_t tile_m, int32_t tile_n,
                               uint64_t* mask_dev, int32_t* skip_dev, void* stream);

/* Launches a one-CTA kernel that waits, with a short limit (`limit_cycles` SM
 * cycles), on a barrier that nothing arrives on, to show that a wait that runs
 * out sets *status_dev and returns instead of hanging.  Mirrors the
 * non-blocking BarrierTryWait contract (include/axp/realize/sm90.hpp:1300-1322). */
int axp_sm100_selftest_bounded_wait(int64_t limit_cycles, void* stream, uint32_t* status_dev);

/* Process-wide tuning option; value 0 restores the library default.
 *   "gemm.epilogue_warpgroups"  2 or 4: warpgroups that drain the accumulator
 *   "gemm.cta_group"            1 or 2: CTAs cooperating on one MMA (2 = cluster pair, the default for both GEMMs:
 *                               256 x 256 tile per pair, each CTA loads its own operand halves; the E4M3 gate / up
 *                               (SwiGLU) GEMM runs single CTAs unless 2 is chosen)
 *   "gemm.fp8_tile"             FP8 block-scaled GEMM: 256 = 128 x 256 tiles per CTA (default); 128 = 128 x 128
 *                               tiles with two CTAs per SM (same results bit for bit; measured 13 % slower on 8192^3)
 *   "attn.exp_mode"             how the softmax exponentials are evaluated: 1 = all on the SFU;
 *                               2 / 3 / 4 = 2 / 4 / 3 of every 8 pairs as a polynomial on the FMA pipe
 *   "attn.p_operand"            E4M3 attention: 1 = P reaches the P.V MMA in tensor memory,
 *                               2 = through shared memory (the next Q.K^T then overlaps the softmax)
 *   "attn.rescale"              prefill attention: when a row's reference maximum advances.  1 = on every new maximum
 *                               (the standard online softmax; P <= 1, the largest weight of a tile is exact in E4M3);
 *                               2 = lazily, when a tile maximum exceeds it by more than 2^8 (the default: 13-15 % faster;
 *                               for E4M3 P the rounding noise against exact attention is about 1.7 times the standard
 *                               rule's on peaked softmax rows, for bf16 P there is no measurable difference)
 *   "attn.kv_tile"              bf16 attention: 64 or 128 keys per KV tile (64: two S buffers per Q tile in
 *                               tensor memory, the next Q.K^T never waits for the softmax)
 *   "attn.issuers"              1 or 2 threads issuing the attention MMAs (2: one per Q tile)
 *   "attn.decode_kernel"        split-KV calls with at most 16 query rows per KV head: 1 = the forward kernel,
 *                               2 = the decode kernel with swapped operands (keys on the tensor-memory lanes)
 * Two more names, "debug_buffer" and "gemm.experiment", belong to the latency probes of builds made with
 * -DAXP_SM100_LATENCY_PROBES (globaltimer stamps, parts of the epilogue switched off; results are then not
 * valid); the production library answers AXP_ERR_UNSUPPORTED for them and its kernels carry none of that code.
 * The counterpart upstream is the expert override traits of the intent selectors
 * (include/axp/kits/intent.hpp:108-125), which are compile-time. */
int axp_sm100_set_option(const char* name, int64_t value);

/* Thread-local description of the last failure reported on this thread. */
const char* axp_sm100_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* AXP_SM100_H_ */
