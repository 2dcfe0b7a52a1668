/* rtxb — C ABI of the sm_100a block-scaled quantize + GEMM kernels.
 *
 * The reference (achiya-deri-work/rtx) has no FFI: its seam is a set of Python
 * `compile_*` factories that return launch callables `(tensors...) -> None`
 * running asynchronously on the current CUDA stream.  Each entry point below
 * replaces one of those callables; the citation names the factory and the
 * call sites that bind it.
 *
 * Conventions (all entry points)
 *   - plain device pointers and sizes; no allocation, no synchronisation, no
 *     exceptions; work is enqueued on `stream` (a cudaStream_t passed as void*)
 *     of the device that is current;
 *   - returns 0 (RTXB_OK) or a negative RTXB_E_* code; rtxb_error_string()
 *     explains it; a rejected call has launched nothing;
 *   - payload matrices are K-major (row-major [rows, K] with K contiguous),
 *     BF16 inputs may have a row pitch `ld` (elements) >= K;
 *   - `status` is an optional device int the kernels set to a non-zero
 *     RTXB_DEV_* code when a bounded wait runs out (they then leave through
 *     their normal teardown); the caller zeroes and reads it;
 *   - scale layouts use the reference's codes (rtx/formats/common.py:17):
 *     0 = row_major [rows, blocks], 2 = mma128 (128-row tiles of 512 bytes,
 *     byte (row%32)*16 + ((row/32)%4)*4 + block%4, tiles ordered
 *     [row/128][block/4]); 1 = mma64 is an SM120-only layout and is rejected.
 */
#ifndef RTXB_H_
#define RTXB_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RTXB_OK 0
#define RTXB_E_INVALID_ARGUMENT (-1)
#define RTXB_E_UNSUPPORTED (-2)
#define RTXB_E_ALIGNMENT (-3)
#define RTXB_E_WORKSPACE (-4)
#define RTXB_E_CUDA (-5)
#define RTXB_E_DRIVER (-6)
#define RTXB_E_SCRATCH_CAPACITY (-7)

#define RTXB_SCALE_ROW_MAJOR 0
#define RTXB_SCALE_MMA64 1
#define RTXB_SCALE_MMA128 2

#define RTXB_ROUND_FLOOR 0
#define RTXB_ROUND_INFINITY 1

#define RTXB_OUT_BF16 0
#define RTXB_OUT_F32 1

#define RTXB_TENSOR_SCALE_EXACT 0
#define RTXB_TENSOR_SCALE_POWER2 1

/* codes a kernel leaves in the caller's `status` word when one of its bounded waits runs out */
#define RTXB_DEV_OK 0
#define RTXB_DEV_WAIT_PRODUCER 1   /* TMA producer: no free ring slot */
#define RTXB_DEV_WAIT_MMA 2        /* MMA issuer: operands or accumulator columns never arrived */
#define RTXB_DEV_WAIT_EPILOGUE 3   /* epilogue: accumulator never completed */
#define RTXB_DEV_WAIT_QUANT 4      /* in-kernel quantizer warps */
#define RTXB_DEV_WAIT_SELFTEST 5   /* rtxb_selftest_wait_timeout */
#define RTXB_DEV_WAIT_PEER 6       /* rtxb_peer_barrier: another rank's flag never arrived */

int rtxb_version(void);
const char* rtxb_error_string(int code);
/* last CUDA/driver error text recorded by this thread's most recent failing call */
const char* rtxb_last_cuda_error(void);

/* Barrier among the (<= 8) ranks of one node through flag words in peer-mapped memory; every rank calls it on its
 * own GPU, the same number of times.  No counterpart in the reference (single GPU).  rank_flags[t] is rank t's
 * array of 8 int32 words, mapped into this process; epoch_counter is one int32 of this rank's own device memory
 * that the kernel advances (the launch carries no per-call number, so it can be replayed from a captured
 * graph); all of them zero before the first barrier.  Work enqueued before the call on `stream`, including stores into other ranks' memory, is
 * visible to every rank's work enqueued after its own call.  Each wait is bounded by `limit_ns` (1 ms .. 2 s): if a
 * rank never arrives, RTXB_DEV_WAIT_PEER is stored in `status` and the kernel returns. */
int rtxb_peer_barrier(void* const* rank_flags, int world, int rank, int* epoch_counter, int64_t limit_ns,
                      void* stream, int* status);

/* Self-test of the failure path every kernel role shares.  No counterpart in the reference.  Launches one warp
 * that waits, with the bounded wait the GEMM and quantizer roles use, on a barrier that nothing completes; after
 * `limit_ns` nanoseconds (1 ms .. 2 s) the wait gives up, the kernel stores RTXB_DEV_WAIT_SELFTEST in `status`
 * (and the time it waited in `waited_ns`, optional) and returns normally: the context stays usable and the next
 * launch runs.  This is how a lost arrival reaches the host, instead of a hung GPU. */
int rtxb_selftest_wait_timeout(int64_t limit_ns, void* stream, int* status, unsigned long long* waited_ns);

/* SMs that the persistent kernels of this library leave unused from now on (process-wide; 0 =
 * use every SM).  No counterpart in the reference (single GPU): the GEMMs here hold every SM for
 * their whole run, so a collective that should overlap one (the NCCL all-reduce of dW beside the dX
 * GEMM) only gets to run if some SMs are left to it. */
int rtxb_set_sm_margin(int sms);
int rtxb_get_sm_margin(void);

/* GEMM schedule used by the calls this thread makes from now on.  The reference selects a schedule per
 * call through the config object given to its compile_* factories (tile shape, stages, persistence:
 * rtx/configs/mxfp8.py:110-343, chosen by rtx/autotune); here the built schedules are an enumeration:
 * AUTO (the library picks by shape), SINGLE (one CTA per 128 x 256 tile, 4 stages), PAIR (two CTAs per
 * 256 x 256 tile, cta_group::2), STREAM (128 x 64 tiles for M <= 128; ignored for larger M), FUSED_X (the
 * composite MXFP8 forwards skip the activation quantizer launch and run the pair kernel whose own
 * quantizer warps encode X tile by tile, rtxb_mxfp8_linear_fwd_fused_x; packed-operand GEMMs treat it
 * as PAIR).  All give the same bits.
 * The setting is a property of the calling THREAD, read when a call is made: it is safe across threads
 * and streams, but a caller that sets it around a call must restore it itself, and nested users on one
 * thread see each other's setting (set it immediately before the call it is meant for). */
#define RTXB_SCHEDULE_AUTO 0
#define RTXB_SCHEDULE_SINGLE 1
#define RTXB_SCHEDULE_PAIR 2
#define RTXB_SCHEDULE_STREAM 3
#define RTXB_SCHEDULE_FUSED_X 4
int rtxb_set_gemm_schedule(int schedule);
int rtxb_get_gemm_schedule(void);

/* ---- sizes ------------------------------------------------------------- */

/* padded K: 32-multiples (rtx/kernels/mxfp8.py:57-66, rtx/configs/nvfp4.py:15-28) */
int64_t rtxb_mxfp8_storage_k(int64_t k);
int64_t rtxb_nvfp4_storage_k(int64_t k);
/* bytes of a scale buffer for `rows` x `k` in `layout` (mma128 includes row and K padding) */
size_t rtxb_mxfp8_scale_bytes(int64_t rows, int64_t k, int layout);
size_t rtxb_nvfp4_scale_bytes(int64_t rows, int64_t k, int layout);

/* ---- MXFP8 quantizers ---------------------------------------------------
 * compile_mxfp8_quant(rows, k, cfg) -> (src bf16, q e4m3[R,Kp], s e8m0)
 *   rtx/kernels/mxfp8_quant.py:52-395; bound at rtx/fp8.py:783-786, :930-931.
 * compile_mxfp8_transposed_quant -> same outputs for the logical transpose of a
 *   stored [K, R] matrix: rtx/kernels/mxfp8_quant.py:526-1019; rtx/fp8_bwd.py:437-448. */
int rtxb_mxfp8_quantize(const void* src_bf16, int64_t rows, int64_t k, int64_t ld, void* q, void* scales,
                        int scale_layout, int rounding, void* stream);
int rtxb_mxfp8_quantize_transposed(const void* src_bf16_k_by_rows, int64_t rows, int64_t k, int64_t ld, void* q,
                                   void* scales, int scale_layout, int rounding, void* stream);

/* compile_mxfp8_backward_quad_quant(..., shared_g=True) reads the gradient once for its two
 * quantizations (rtx/kernels/mxfp8_quant.py:1400-1763; bound at rtx/fp8_bwd.py:545-555).  Here:
 * src [m, n] -> q_rows [m, np] with scales along n (= rtxb_mxfp8_quantize) AND q_t [n, mp] with
 * scales along m (= rtxb_mxfp8_quantize_transposed), both from one staged read of src. */
int rtxb_mxfp8_quantize_dual(const void* src_bf16, int64_t m, int64_t n, int64_t ld, void* q_rows, void* s_rows,
                             void* q_t, void* s_t, int scale_layout, int rounding, void* stream);
/* ---- MXFP8 GEMM on packed operands ---------------------------------------
 * compile_mxfp8_gemm(problem, cfg, ...) -> (qx, qw, sx, sw, out)
 *   rtx/kernels/mxfp8_gemm.py:2048-2151; bound at rtx/fp8.py:932, :1260, :1338 and
 *   rtx/fp8_bwd.py:458-505.  out[m, n] = bf16 or f32 of sum_k deq(qa) deq(qb)^T.
 * Scales must be in the mma128 layout.  `k` is the logical K; rows of qa/qb are
 * rtxb_mxfp8_storage_k(k) bytes apart. */
int rtxb_mxfp8_gemm(const void* qa, const void* sa, const void* qb, const void* sb, void* out, int64_t m, int64_t n,
                    int64_t k, int64_t ldo, int out_dtype, void* stream, int* status);
/* The same GEMM with its output split into n_blocks (<= 8) blocks of `block_rows` rows (a multiple of 256, the
 * last block may be shorter), block j written to out_blocks[j] (a [rows, n] matrix of pitch ldo, 16-byte aligned).
 * No counterpart in the reference (single GPU).  The buffers may live on other GPUs of the node (peer-mapped
 * addresses): the epilogue's TMA stores then travel over NVLink while the MMAs of the next tile run, which is how
 * the data-parallel backward turns the reduce-scatter of dW into the GEMM's own output traffic.  The tile order
 * starts at the tiles of block `first_block` so that ranks writing to one another begin at different owners.
 * CTA-pair kernel only (m >= 256). */
int rtxb_mxfp8_gemm_row_blocks(const void* qa, const void* sa, const void* qb, const void* sb, void* const* out_blocks,
                               int n_blocks, int64_t block_rows, int64_t m, int64_t n, int64_t k, int64_t ldo,
                               int out_dtype, int first_block, void* stream, int* status);
/* SwiGLU gate/up projection with the activation fused into the epilogue:
 * qb holds [2*inter, K] (gate rows first); out bf16 [m, inter] =
 * silu(acc[:, :inter]) * acc[:, inter:], one BF16 rounding.  The reference
 * computes this as linear + chunk + F.silu * up (rtx/models/decoder.py:382-384).
 * inter must be a multiple of 128. */
int rtxb_mxfp8_gemm_glu(const void* qa, const void* sa, const void* qb, const void* sb, void* out_bf16, int64_t m,
                        int64_t inter, int64_t k, int64_t ldo, void* stream, int* status);

/* The same GEMM whose epilogue also quantizes H for the next projection: q_h e4m3 [m, inter] and
 * s_h (E8M0, mma128 tiles) are bit-identical to rtxb_mxfp8_quantize applied to the BF16 H (each
 * 32-column group a thread holds is one MX block).  h_bf16 may be NULL when only the packed H is
 * needed; that removes a BF16 write and read of H and one quantizer launch from the MLP. */
int rtxb_mxfp8_gemm_glu_mx(const void* qa, const void* sa, const void* qb, const void* sb, void* h_bf16, void* q_h,
                           void* s_h, int64_t m, int64_t inter, int64_t k, int64_t ldo, void* stream, int* status);

/* ---- fused forward (quantize both operands + GEMM) ------------------------
 * compile_mxfp8_fwd(problem, cfg) -> (x bf16, w bf16, out bf16[M,N])
 *   rtx/kernels/mxfp8_fwd.py:2963-3029; bound at rtx/fp8.py:560, :581, :635.
 * and the materialized pair compile_mxfp8_dual_quant + compile_mxfp8_gemm run by
 *   _PrequantRunner (rtx/fp8.py:292-312).
 * Two launches on `stream`: one quantizer launch for both operands, then the GEMM as a programmatic dependent of
 * it (the GEMM waits for the quantizer's grid before its first operand load).
 * workspace: rtxb_mxfp8_linear_workspace_bytes(m, n, k); caller-owned, reusable
 * across calls on the same stream. */
size_t rtxb_mxfp8_linear_workspace_bytes(int64_t m, int64_t n, int64_t k);
/* The reference's fused forward kernel MXFP8FusedLinearKernel (rtx/kernels/mxfp8_fwd.py:936-2934: BF16
 * tiles staged, quantizer warps, MMA, one launch) for the operand state "dynamic X, packed W"
 * (op mxfp8_linear_dynamic_x_prequant_w, rtx/fp8.py:1269-1302): x stays BF16 in memory and is quantized
 * tile by tile by the GEMM's quantizer warps; qw / sw are the packed weight [n, Kp] and its mma128
 * scales.  Bit-identical to rtxb_mxfp8_quantize(x) followed by rtxb_mxfp8_gemm.  Every 256-wide column
 * tile re-quantizes its rows of x, so this pays only where n is a few tiles wide. */
int rtxb_mxfp8_linear_fwd_fused_x(const void* x_bf16, int64_t ldx, const void* qw, const void* sw, void* out_bf16,
                                  int64_t m, int64_t n, int64_t k, int64_t ldo, int rounding, void* stream, int* status);
/* rtxb_mxfp8_gemm_glu_mx with the same in-kernel quantization of the activation operand. */
int rtxb_mxfp8_gemm_glu_mx_fused_x(const void* x_bf16, int64_t ldx, const void* qb, const void* sb, void* h_bf16,
                                   void* q_h, void* s_h, int64_t m, int64_t inter, int64_t k, int64_t ldo, void* stream,
                                   int* status);
int rtxb_mxfp8_linear_fwd(const void* x_bf16, const void* w_bf16, void* out_bf16, int64_t m, int64_t n, int64_t k,
                          int rounding, void* workspace, size_t workspace_bytes, void* stream, int* status);

/* The same forward with no scratch argument, for callers that cannot allocate.
 * (No counterpart in the reference, whose runners allocate their workspaces with
 * PyTorch.)  Meant for hosts that only hold the input and output buffers they were
 * given — generated wrappers calling `launcher(x, w, out=buf)`, plugins inside another
 * runtime's memory pool, sections where cudaMalloc's device-wide synchronisation is
 * not acceptable.  The quantized operands go to a fixed RTXB_NOALLOC_SCRATCH_BYTES
 * array that is part of the library image on every GPU that loads it; the call
 * allocates and frees nothing.
 *   - Shapes whose operands need more than that array (the value
 *     rtxb_mxfp8_linear_workspace_bytes(m, n, k) reports) are refused with
 *     RTXB_E_SCRATCH_CAPACITY and nothing is launched.
 *   - The first call on each device looks up that device's address of the array
 *     (the device must be current, as for every entry point); make that first call
 *     before starting any stream capture.  `stream` must belong to the current device:
 *     a stream of another device is refused (RTXB_E_INVALID_ARGUMENT), since the
 *     kernels would run there with this device's address of the array.
 *   - All calls on a device share the one array and it keeps the last call's
 *     contents.  Nothing in it needs clearing between calls (each call rewrites all
 *     it reads), but two calls whose kernels overlap on the GPU — different streams
 *     without an ordering between them — race on it.  Order them. */
#define RTXB_NOALLOC_SCRATCH_BYTES (32 * 1024 * 1024)
int rtxb_mxfp8_linear_fwd_noalloc(const void* x_bf16, const void* w_bf16, void* out_bf16, int64_t m, int64_t n,
                                  int64_t k, int rounding, void* stream, int* status);

/* SwiGLU MLP forward: H = silu(X Wg^T) * (X Wu^T), Y = H Wd^T, every GEMM
 * operand MXFP8-quantized along its K.  w_gate_up bf16 [2*inter, k], w_down
 * bf16 [n_out, inter]; y_bf16 [m, n_out] is the output; h_bf16 [m, inter] is an optional output
 * (NULL: H only ever exists in its MXFP8 form, written by the gate/up epilogue).
 * Five launches on `stream`: quantizers of X and W_gate_up, the gate/up GEMM, the quantizer of W_down (a
 * programmatic dependent that runs beside that GEMM), the down GEMM.  All operands must be complete on the stream
 * before the call; none may be written by other streams while it runs. */
size_t rtxb_mxfp8_glu_mlp_workspace_bytes(int64_t m, int64_t k, int64_t inter, int64_t n_out);
int rtxb_mxfp8_glu_mlp_fwd(const void* x_bf16, const void* w_gate_up_bf16, const void* w_down_bf16, void* h_bf16,
                           void* y_bf16, int64_t m, int64_t k, int64_t inter, int64_t n_out, void* workspace,
                           size_t workspace_bytes, void* stream, int* status);

/* ---- MXFP8 backward --------------------------------------------------------
 * _build_bwd_runner / _BwdRunner (rtx/fp8_bwd.py:521-568, :229-325):
 *   dX[M,K] = dY[M,N] W[N,K]   (operands quantized along N)
 *   dW[N,K] = dY^T[N,M] X[M,K] (operands quantized along M)
 * dx is BF16; dw is BF16 (reference dtype) or FP32 (for a data-parallel
 * all-reduce) per dw_dtype.  Either output may be NULL to skip that product. */
size_t rtxb_mxfp8_backward_workspace_bytes(int64_t m, int64_t n, int64_t k);
int rtxb_mxfp8_linear_bwd(const void* dy_bf16, const void* x_bf16, const void* w_bf16, void* dx_bf16, void* dw,
                          int dw_dtype, int64_t m, int64_t n, int64_t k, void* workspace, size_t workspace_bytes,
                          void* stream, int* status);

/* compile_mxfp8_workspace_reduce(m, n, split, algorithm="serial", ...) -> (ws f32 [split, m, n], out bf16)
 *   rtx/kernels/mxfp8_reduce.py:20-104; bound at rtx/fp8_bwd.py:351-386, :464-495.
 * out[i] = bf16(parts[0][i] + parts[1][i] + ...), parts `part_stride` floats apart, summed in index order and
 * rounded once.  The reference reduces the partial tiles of its split-K GEMMs with it; here it sums the per-rank
 * FP32 blocks of dW that the data-parallel backward collects in the owner's staging slots. */
int rtxb_sum_parts_f32_to_bf16(const float* parts, int n_parts, int64_t part_stride, int64_t count, void* out_bf16,
                               void* stream);

/* ---- NVFP4 -----------------------------------------------------------------
 * Outer scale: the reference computes it with PyTorch reductions
 * (_outer_tensor_scale, rtx/fp4.py:343-365).  rtxb_nvfp4_tensor_scale does the
 * |max| reduction and the scale rule on the device: scale_out[0] = scale;
 * when other_scale/out_scale are non-NULL also out_scale[0] = scale * other_scale[0].
 * amax_scratch: 4 bytes of device memory. */
int rtxb_nvfp4_tensor_scale(const void* src_bf16, int64_t rows, int64_t k, int64_t ld, int mode, void* amax_scratch,
                            float* scale_out, const float* other_scale, float* out_scale, void* stream);
/* compile_nvfp4_quant(rows, k, cfg) -> (src bf16, q u8[R,Kp/2], s e4m3, tensor_scale f32[1])
 *   rtx/kernels/nvfp4_quant.py:32-349; bound at rtx/fp4.py:696-697, :900, :1532.
 * tensor_scale NULL = block policy (scale 1.0, compile_nvfp4_block_quant). */
int rtxb_nvfp4_quantize(const void* src_bf16, int64_t rows, int64_t k, int64_t ld, void* q, void* scales,
                        int scale_layout, const float* tensor_scale, void* stream);
/* Outer scale + quantization of one tensor with the scale taken from its own current |max|
 * (NVFP4Linear.forward with scaling="current": _outer_tensor_scale, rtx/fp4.py:343-365, then
 * compile_nvfp4_quant).  Same results as rtxb_nvfp4_tensor_scale followed by rtxb_nvfp4_quantize;
 * tensors of at most 64 tiles of 128 x 256 values (decode activations) take two launches chained
 * by programmatic dependent launch (per-CTA |max| partials, then scale rule + quantization in
 * every CTA; no memset, no finalize launch), larger ones the three launches.
 * amax_scratch: 256 bytes of device memory, 4-byte aligned. */
int rtxb_nvfp4_quantize_dynamic(const void* src_bf16, int64_t rows, int64_t k, int64_t ld, int mode, void* q,
                                void* scales, int scale_layout, float* scale_out, const float* other_scale,
                                float* out_scale, void* amax_scratch, void* stream);
/* ---- NVFP4 delayed policy (scaling="delayed") --------------------------------------------
 * compile_nvfp4_delayed_dual_quant(...) -> (x, w, qx, qw, sx, sw, x_history, weight_history,
 * next_x_history, next_weight_history, output_scale); kernel NVFP4DelayedDualQuantKernel,
 * rtx/kernels/nvfp4_quant.py:473-664; bound at rtx/fp4.py:736; runner _DelayedDynamicRunner
 * rtx/fp4.py:462-517.  Per operand here: the outer scale is the tensor-scale rule applied to
 * max(history[0 .. len)) (window_max != 0) or to history[0] (most recent); the tensor is quantized
 * with it in the same single read that observes its |max|; next_history[0] = observed |max|,
 * next_history[i] = history[i - 1].  history_len is 1, 4, 16 or 64; the two generations must not
 * alias.  scale_out[0] = the scale used; with other_scale / out_scale also the product. */
int rtxb_nvfp4_quantize_delayed(const void* src_bf16, int64_t rows, int64_t k, int64_t ld, void* q, void* scales,
                                int scale_layout, const float* history, float* next_history, int history_len,
                                int window_max, int mode, float* scale_out, const float* other_scale, float* out_scale,
                                void* stream);
/* Both operands + GEMM; workspace as rtxb_nvfp4_linear_workspace_bytes(m, n, k). */
int rtxb_nvfp4_linear_fwd_delayed(const void* x_bf16, const void* w_bf16, void* out_bf16, int64_t m, int64_t n,
                                  int64_t k, const float* x_history, const float* w_history, float* next_x_history,
                                  float* next_w_history, int history_len, int window_max, int scale_mode,
                                  void* workspace, size_t workspace_bytes, void* stream, int* status);

/* ---- NVFP4 row-region policy (scaling="jit_row_region", the reference's default) ----------
 * compile_nvfp4_jit_region_dual_quant(x_rows, weight_rows, k, cfg, x_region_rows, weight_region_rows,
 * tensor_scale_mode, ...) -> (x, w, qx, qw, sx, sw, region_scales)   rtx/kernels/nvfp4_quant.py:1623-1678,
 * kernel NVFP4JITRegionDualQuantKernel :667-1000; bound at rtx/fp4.py:817-830.
 * One FP32 outer scale per `region_rows` consecutive rows, the tensor-scale rule applied to the
 * region's current |max|.  Here per operand: rtxb_nvfp4_region_scales (one warp per region; a single
 * region = the whole tensor takes the grid-wide reduction and needs the 4-byte amax_scratch), then
 * rtxb_nvfp4_quantize_regions.  region_rows must divide rows. */
int rtxb_nvfp4_region_scales(const void* src_bf16, int64_t rows, int64_t k, int64_t ld, int64_t region_rows, int mode,
                             void* amax_scratch, float* scales_out, void* stream);
int rtxb_nvfp4_quantize_regions(const void* src_bf16, int64_t rows, int64_t k, int64_t ld, void* q, void* scales,
                                int scale_layout, const float* region_scales, int64_t region_rows, void* stream);
/* compile_nvfp4_jit_region_gemm(problem, cfg, x_region_rows, weight_region_rows) ->
 * (qx, qw, sx, sw, out bf16, region_scales)   rtx/kernels/nvfp4_gemm.py; epilogue
 * rtx/kernels/mxfp8_gemm.py:1720-1760: out[m,n] = bf16(acc * (xs[m / Rx] * ws[n / Rw])). */
int rtxb_nvfp4_gemm_regions(const void* qa, const void* sa, const void* qb, const void* sb, void* out_bf16, int64_t m,
                            int64_t n, int64_t k, int64_t ldo, const float* x_region_scales, int64_t x_region_rows,
                            const float* w_region_scales, int64_t w_region_rows, void* stream, int* status);
/* _JITRegionDynamicRunner (rtx/fp4.py:522-560, built at :758-845).  Region sizes are requests: one
 * that does not split the operand's rows evenly into more than one region falls back to a single
 * region over the tensor (rtx/fp4.py:89-94).  Five launches (region scales and quantizer per operand, GEMM); where
 * both operands' regions are small (below 32 KB) three: the two operands share the region-scale launch and the
 * quantizer launch, and the GEMM follows as a programmatic dependent. */
size_t rtxb_nvfp4_linear_regions_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t x_region_rows,
                                                 int64_t w_region_rows);
int rtxb_nvfp4_linear_fwd_regions(const void* x_bf16, const void* w_bf16, void* out_bf16, int64_t m, int64_t n,
                                  int64_t k, int64_t x_region_rows, int64_t w_region_rows, int scale_mode,
                                  void* workspace, size_t workspace_bytes, void* stream, int* status);
/* compile_nvfp4_gemm(problem, cfg) -> (qx, qw, sx, sw, out bf16, output_scale f32[1])
 *   rtx/kernels/nvfp4_gemm.py:22-64, epilogue rtx/kernels/mxfp8_gemm.py:779-781;
 *   bound at rtx/fp4.py:707, :901, :1734, :2313.  output_scale NULL = 1 (block GEMM). */
int rtxb_nvfp4_gemm(const void* qa, const void* sa, const void* qb, const void* sb, void* out, int64_t m, int64_t n,
                    int64_t k, int64_t ldo, int out_dtype, const float* output_scale, void* stream, int* status);
/* _DynamicRunner (rtx/fp4.py:404-454): outer scales + dual quantize + GEMM. */
size_t rtxb_nvfp4_linear_workspace_bytes(int64_t m, int64_t n, int64_t k);
int rtxb_nvfp4_linear_fwd(const void* x_bf16, const void* w_bf16, void* out_bf16, int64_t m, int64_t n, int64_t k,
                          int scale_mode, void* workspace, size_t workspace_bytes, void* stream, int* status);

/* _DynamicXRunner (rtx/fp4.py:639-668) behind the op nvfp4_linear_dynamic_x_prequant_w
 * (rtx/fp4.py:1628-1686), with the activation's outer scale taken from its current |max| in the
 * same call: x BF16 [M,K]; qw / sw the packed weight [N, Kp/2] and its mma128 block scales;
 * w_scale its FP32 outer scale (device scalar).  Three launches for decode-sized M (|max|
 * partials, quantizer, GEMM), each a programmatic dependent of the one before: the GEMM streams
 * the weights into shared memory while the activations are still being quantized.  The packed weight must therefore
 * be complete before this call is enqueued (any earlier work on the stream is fine). */
size_t rtxb_nvfp4_linear_prequant_w_workspace_bytes(int64_t m, int64_t k);
int rtxb_nvfp4_linear_fwd_prequant_w(const void* x_bf16, const void* qw, const void* sw, const float* w_scale,
                                     void* out_bf16, int64_t m, int64_t n, int64_t k, int scale_mode, void* workspace,
                                     size_t workspace_bytes, void* stream, int* status);

#ifdef __cplusplus
}
#endif
#endif /* RTXB_H_ */
