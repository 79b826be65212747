/* gnf4b.h -- C ABI of libgnf4b.so: grouped 4-bit expert GEMM for NVIDIA B200 (sm_100a).
 *
 * One shared library, plain pointers and sizes, no framework types.  Every
 * pointer is a DEVICE pointer unless its comment says "host".  Every launch
 * goes to the CUDA stream passed as `cuda_stream` (a cudaStream_t cast to
 * void*; NULL = the legacy default stream) and returns without synchronising.
 * Functions return 0 on success and a negative GNF4B_E* code on a contract
 * violation; nothing aborts and no kernel traps.
 *
 * Each entry point names the interface of the reference project
 * (pjordanandrsn/grouped-nf4-gemm v0.13.2, paths relative to its root) that it
 * stands in for.
 */
#ifndef GNF4B_H_
#define GNF4B_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GNF4B_ABI_VERSION 1

/* weight formats */
#define GNF4B_FMT_NF4   0   /* bitsandbytes NF4: element 2j = HIGH nibble, absmax per 64 */
#define GNF4B_FMT_MXFP4 1   /* OCP MXFP4: element 2j = LOW nibble, e8m0 scale per 32    */
/* operations */
#define GNF4B_OP_FWD    0   /* out[T,N] = x[T,K] . W[e]^T   (contract over K) */
#define GNF4B_OP_DGRAD  1   /* out[T,K] = x[T,N] . W[e]     (contract over N) */
/* activation dtypes */
#define GNF4B_X_BF16    0
#define GNF4B_X_FP16    1
/* scale dtypes */
#define GNF4B_S_F32     0   /* NF4 absmax, fp32                                  */
#define GNF4B_S_BF16    1   /* NF4 absmax stored as bf16 (widened exactly)       */
#define GNF4B_S_E8M0    2   /* MXFP4 block exponent byte, value 2^(e-127)        */

/* flags */
#define GNF4B_PATH_AUTO    0u
#define GNF4B_PATH_STREAM  1u   /* CUDA-core streaming kernel (decode-sized groups)   */
#define GNF4B_PATH_TENSOR  2u   /* tcgen05 / TMEM kernel (prefill-sized groups)       */
#define GNF4B_PATH_MASK    3u
#define GNF4B_SPLITK_SHIFT 8    /* bits 8..15: forced split-K factor, 0 = planner     */
#define GNF4B_SPLITK_MASK  0xff00u
#define GNF4B_FLAG_CTA_PAIR      0x20000u /* forward tensor kernel as CTA pairs (cta_group::2 MMAs, each CTA
                                            loads half of the activation tile); default: single CTAs */
#define GNF4B_FLAG_SMEM_OPERANDS 0x10000u /* ablation: forward on the first tensor kernel (both MMA
                                            operands in shared memory) instead of weights in TMEM */

#define GNF4B_FLAG_TABLES_READY   0x40000u /* group_offsets / expert_ids were not written by the kernel launched
                                            just before this call on the stream (they were uploaded, or made
                                            earlier): the decode kernel then streams its first weights while
                                            that previous kernel is still running */
#define GNF4B_FLAG_DECODE_ONE_ROW 0x80000u /* ablation: decode kernel with one weight row per warp in flight where it
                                            would keep two */

#define GNF4B_FLAG_DECODE_BF16_ROWS 0x2000000u /* ablation: decode kernel, two activation rows per pass kept as bf16 pairs
                                               and widened on use where it would keep them as fp32 (NF4, K <= 1024) */
#define GNF4B_FLAG_FFN_UNFUSED    0x100000u /* ablation: gnf4b_ffn_grouped as three launches even where one fused
                                             launch would be taken */
/* x is the gate_up output of the expert FFN, bf16 [T, 2K], and the activation between the two GEMMs is applied while
 * its rows are loaded: SiLU(x[:, :K]) * x[:, K:] (the arithmetic of gnf4b_silu_glu), or the gpt-oss form on
 * interleaved columns (gnf4b_glu_gpt_oss without bias).  Saves the activation launch and its pass over memory; same
 * bits as the two-launch form.  Forward only, on the decode kernel (small groups: max_rows given and <= 16);
 * GNF4B_EUNSUPPORTED otherwise -- the caller then runs the activation kernel itself. */
#define GNF4B_FLAG_SPARSE_GROUPS 0x1000000u /* the caller expects most groups of the list to be empty (a fixed-size list
                                              with the used groups first, padding behind): the decode kernel then deals
                                              out only the groups that exist, so that all SMs share them */
#define GNF4B_FLAG_HOST_COPIES   0x800000u  /* ablation, host-buffer entry points: move a small call's inputs and result
                                              with the copy engines even where two small kernels would do it */
#define GNF4B_FLAG_X_SILU_GLU    0x200000u
#define GNF4B_FLAG_X_GPT_OSS_GLU 0x400000u
/* activations of gnf4b_ffn_grouped */
#define GNF4B_ACT_SILU_GLU    0   /* SiLU(gate) * up, gate = the first half of the gate_up columns            */
#define GNF4B_ACT_GPT_OSS_GLU 1   /* gpt-oss: gate / up interleaved, clamped at 7, (up+1) * gate * sigmoid(1.702 gate) */

/* error codes */
#define GNF4B_OK            0
#define GNF4B_EINVAL       -1   /* bad enum / null pointer / negative size            */
#define GNF4B_ESHAPE       -2   /* K not a multiple of the quant block, N<=0, ...     */
#define GNF4B_EWORKSPACE   -3   /* workspace missing or too small                     */
#define GNF4B_ECUDA        -4   /* a CUDA runtime call failed (see gnf4b_last_cuda_error) */
#define GNF4B_EUNSUPPORTED -5   /* combination not built (e.g. fp16 x on the tensor path) */
#define GNF4B_ETOOBIG      -6   /* size beyond a stated fixed maximum                 */

/* bits a kernel may OR into *status_word (device int32) */
/* expert_ids[g] == GNF4B_PAD_EXPERT marks a padding group: its rows are skipped (the output rows are left
 * untouched) and nothing is flagged.  Lets a caller leave gaps in the row matrix -- e.g. unused capacity of a
 * fixed-size exchange buffer -- without compacting it.  The reference has no such id (its ids are always valid). */
#define GNF4B_PAD_EXPERT (-1)
#define GNF4B_ST_BAD_EXPERT  1  /* an expert id outside [0,E) was skipped             */
#define GNF4B_ST_BAD_OFFSETS 2  /* group_offsets not monotone / beyond T; group skipped */
#define GNF4B_ST_TIMEOUT     4  /* a bounded device-side wait gave up                 */

int gnf4b_abi_version(void);
const char* gnf4b_strerror(int rc);
/* text of the last CUDA error seen by this library on the calling thread */
const char* gnf4b_last_cuda_error(void);

/* The grouped GEMM.  Stands in for the launches inside
 *   gemm_4bit_grouped   kernel/nf4_grouped.py:697-907  (fmt NF4,  op FWD)
 *   dgrad_4bit_grouped  kernel/nf4_grouped.py:1056-1121 (fmt NF4, op DGRAD)
 *   gemm_mxfp4_grouped  kernel/mxfp4_grouped.py:134-172 (fmt MXFP4, op FWD)
 * and for their Triton kernels (_gemv_nf4_grouped[_splitk], _gemm_nf4_grouped,
 * _dgrad_nf4_grouped, _gemv_mxfp4_grouped, _gemm_mxfp4_grouped).
 *
 *   x            [T, K] (FWD) or [T, N] (DGRAD), row-major contiguous, rows sorted by group
 *   W            packed nibbles, logical [E, N, K/2]; byte strides w_stride_e, w_stride_n,
 *                last dimension contiguous.  16-byte aligned base and strides take the
 *                TMA loader, anything else a plain-load producer (same results).
 *   S            scales, logical [E, N, K/64] (NF4) or [E, N, K/32] (MXFP4); ELEMENT strides
 *   group_offsets[G+1] int32, exclusive prefix sum of the group sizes (zero-size groups allowed)
 *   expert_ids   [G] int32, index into the stack handed in (may repeat, any order)
 *   max_rows     largest group size if the host knows it, else <= 0.  Steers the choice of kernel:
 *                with it the streaming kernels are taken up to a mean of 2 to 4 rows per group (by
 *                shape), without it up to 1.5.  It must not be understated: the decode kernel visits
 *                max_rows rows of a group, rows beyond that are NOT computed and the call raises
 *                GNF4B_ST_BAD_OFFSETS.  The kernels agree to bf16 rounding, not to the bit; pin
 *                GNF4B_PATH_* where bit-identical results across calls matter
 *   out          bf16 [T, N] (FWD) or [T, K] (DGRAD)
 *   workspace    device scratch of at least gnf4b_workspace_bytes(...) bytes (may be NULL
 *                when that is 0); must be zero-filled once before its first use, the
 *                kernels leave it zeroed again
 *   status_word  optional device int32 that kernels OR GNF4B_ST_* bits into
 */
int gnf4b_gemm_grouped(int fmt, int op,
                       const void* x, int x_dtype, int64_t T,
                       const uint8_t* W, int64_t w_stride_e, int64_t w_stride_n,
                       const void* S, int s_dtype, int64_t s_stride_e, int64_t s_stride_n,
                       const int32_t* group_offsets, const int32_t* expert_ids,
                       int32_t G, int32_t E, int64_t N, int64_t K, int32_t max_rows,
                       void* out, void* workspace, size_t workspace_bytes,
                       int32_t* status_word, uint32_t flags, void* cuda_stream);

/* Largest scratch gnf4b_gemm_grouped_noalloc can serve (bytes of the built-in device array). */
#define GNF4B_NOALLOC_SCRATCH_BYTES (8u << 20)

/* The same grouped GEMM for callers that cannot allocate device memory.  No counterpart in
 * the reference project: there the split-K scratch is always a fresh torch allocation.
 *
 * Who needs it: code that runs where cudaMalloc is off limits -- inside a region that must
 * not touch the allocator (a serving loop with a frozen memory plan, a plugin hosted by a
 * runtime that owns all device memory and hands out none, a signal-safe or real-time path
 * where an allocation's latency or failure is unacceptable).  Those callers still pass
 * their inputs and the output buffer; only the scratch comes from the library: a
 * file-scope device array of GNF4B_NOALLOC_SCRATCH_BYTES that every GPU loading this
 * library holds until the process exits.
 *
 * Arguments are those of gnf4b_gemm_grouped without workspace / workspace_bytes.
 *   - Returns GNF4B_ETOOBIG when the split-K scratch of this problem
 *     (gnf4b_workspace_bytes) exceeds GNF4B_NOALLOC_SCRATCH_BYTES; nothing is launched.
 *   - Calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - The first call on each device looks the array's device address up
 *     (cudaGetSymbolAddress, with that device current), which with lazy module loading may also
 *     load the module that holds the array; make that first call during warm-up, outside any
 *     CUDA stream capture.
 *   - All calls share the one array and it keeps what the last call left: the part that
 *     must start at zero (the arrival counters) is cleared on `cuda_stream` before every
 *     launch.  Two calls whose kernels overlap on the GPU (different streams, no ordering
 *     between them) race on it; order them.
 */
int gnf4b_gemm_grouped_noalloc(int fmt, int op,
                               const void* x, int x_dtype, int64_t T,
                               const uint8_t* W, int64_t w_stride_e, int64_t w_stride_n,
                               const void* S, int s_dtype, int64_t s_stride_e, int64_t s_stride_n,
                               const int32_t* group_offsets, const int32_t* expert_ids,
                               int32_t G, int32_t E, int64_t N, int64_t K, int32_t max_rows,
                               void* out, int32_t* status_word, uint32_t flags, void* cuda_stream);

/* The grouped GEMM for a caller whose activations, group tables and result live in HOST memory:
 * the signature shape of the reference's native CPU entry points
 *   gnf4_gemv_nf4_grouped    gnf4_native/cpu_kernels.c:751
 *   gnf4_gemv_mxfp4_grouped  gnf4_native/cpu_kernels.c:1097
 *   gnf4_dgrad_nf4_grouped   gnf4_native/cpu_kernels.c:1374
 * (bound through ctypes in gnf4_native/build.py:106-118): host `x`, host `sizes[G]`, host
 * `expert_ids[G]`, host `out`, one blocking call.  The packed stack W / S stays resident on the
 * device (uploading it per call would cost more than the GEMM).
 *
 *   x_host        [T, K] (FWD) or [T, N] (DGRAD), bf16 or fp16, contiguous; pinned memory makes the
 *                 copy asynchronous, pageable memory works
 *   sizes_host    [G] int32 group sizes (zero allowed), sum == T or GNF4B_EINVAL
 *   expert_ids_host [G] int32, each in [0, E) or GNF4B_PAD_EXPERT, else GNF4B_EINVAL (checked on the
 *                 host, nothing is launched)
 *   out_host      bf16 [T, N] (FWD) or [T, K] (DGRAD), all T rows are written; the rows of padding
 *                 groups receive unspecified values (whatever the staging block held)
 *   staging       device scratch of at least gnf4b_host_staging_bytes(...) bytes, 256-byte aligned;
 *                 no initial contents required (the part kernels need zeroed is cleared per call)
 *   status_host   optional host int32: receives the GNF4B_ST_* bits of THIS call
 *
 * What it does on `cuda_stream`: one host-to-device copy of the group tables -- together with `x` when
 * both fit the 64 KiB pinned block the calling thread keeps, else `x` is copied from where it lies --,
 * the launch (the exact largest group size is known here, so the planner's choice is exact), the
 * device-to-host copy of the result, cudaStreamSynchronize.  Not capturable in a CUDA graph (it
 * synchronises).  The first call of a thread allocates its pinned block (cudaHostAlloc); later calls
 * allocate nothing.  Measured on a B200 at the decode shape (8 groups of one row, N=1536, K=2048):
 * 33 us per call, of which the kernel is about 8: the rest is launch, copy-engine and synchronise latency
 * (replacing the two copies by kernels that read and write mapped host memory measured the same).
 */
int gnf4b_gemm_grouped_host(int fmt, int op,
                            const void* x_host, int x_dtype, int64_t T,
                            const uint8_t* W, int64_t w_stride_e, int64_t w_stride_n,
                            const void* S, int s_dtype, int64_t s_stride_e, int64_t s_stride_n,
                            const int32_t* sizes_host, const int32_t* expert_ids_host,
                            int32_t G, int32_t E, int64_t N, int64_t K,
                            void* out_host, void* staging, size_t staging_bytes,
                            int32_t* status_host, uint32_t flags, void* cuda_stream);

/* Device scratch gnf4b_gemm_grouped_host needs: activations, result, group tables, status word and
 * the planner's worst-case workspace for these sizes (any routing of T rows over G groups). */
size_t gnf4b_host_staging_bytes(int fmt, int op, int64_t T, int32_t G, int64_t N, int64_t K, uint32_t flags);

/* One expert FFN per row with host buffers: out = (SiLU(gate) * up) . W_dn[e]^T where
 * [gate | up] = x . W_gu[e]^T (gate = the first N_gu/2 columns, up = the rest).  The GPU counterpart of the
 * reference's fused CPU entry point gnf4_gemv_nf4_ffn_grouped (gnf4_native/cpu_kernels.c:947-986): same
 * operands, host `x`, `sizes`, `expert_ids` and `out`, one blocking call -- here for both weight formats.
 * On `cuda_stream`: one upload (tables, and x when small), the gate_up grouped GEMM, the SiLU-GLU kernel,
 * the down grouped GEMM, one download, one synchronise; the [T, N_gu] intermediate never leaves the device.
 * Results equal gnf4b_gemm_grouped -> gnf4b_silu_glu -> gnf4b_gemm_grouped on the same inputs bit for
 * bit (both intermediates are rounded to bf16).  x must be bf16.  The clamped, interleaved GLU of gpt-oss
 * is not this function's activation.
 *
 *   W_gu / S_gu   gate_up stack, logical [E, N_gu, K_gu/2] and scales; W_dn / S_dn the down stack,
 *                 logical [E, N_dn, (N_gu/2)/2]; both device-resident, one scale dtype for both
 *   out_host      bf16 [T, N_dn]
 *   staging       device scratch of at least gnf4b_ffn_host_staging_bytes(...) bytes, 256-byte aligned
 * Everything else as in gnf4b_gemm_grouped_host. */
int gnf4b_ffn_grouped_host(int fmt, const void* x_host, int x_dtype, int64_t T,
                           const uint8_t* W_gu, int64_t wgu_stride_e, int64_t wgu_stride_n,
                           const void* S_gu, int64_t sgu_stride_e, int64_t sgu_stride_n,
                           const uint8_t* W_dn, int64_t wdn_stride_e, int64_t wdn_stride_n,
                           const void* S_dn, int64_t sdn_stride_e, int64_t sdn_stride_n, int s_dtype,
                           const int32_t* sizes_host, const int32_t* expert_ids_host, int32_t G, int32_t E,
                           int64_t N_gu, int64_t K_gu, int64_t N_dn,
                           void* out_host, void* staging, size_t staging_bytes,
                           int32_t* status_host, uint32_t flags, void* cuda_stream);

size_t gnf4b_ffn_host_staging_bytes(int fmt, int64_t T, int32_t G, int64_t N_gu, int64_t K_gu, int64_t N_dn,
                                    uint32_t flags);

/* One expert FFN per row on DEVICE pointers, on the stream, no synchronisation: out = act(x . W_gu[e]^T) . W_dn[e]^T.
 * The GPU counterpart of the reference's fused CPU FFN gnf4_gemv_nf4_ffn_grouped (gnf4_native/cpu_kernels.c:763-986;
 * its activation is GNF4B_ACT_SILU_GLU) and, with GNF4B_ACT_GPT_OSS_GLU and bias_gu, of the expert path of
 * kernel/mxfp4_pipelined.py:440-445, 453-461 up to the down GEMM (the down bias and the router-weighted sum stay
 * with the caller, in fp32 as there).
 *
 * When every group has one row (max_rows == 1: batch-1 decode), both contractions are at most 3072 long and the
 * stacks are contiguous and 16-byte aligned, it is ONE persistent launch: gate_up GEMV, activation and down GEMV, the
 * [T, N_gu] intermediate crossing L2 only, the down weights streaming into shared memory while gate_up is still
 * being computed.  Otherwise (and with GNF4B_FLAG_FFN_UNFUSED) it is the three launches gnf4b_gemm_grouped ->
 * activation kernel -> gnf4b_gemm_grouped.  Both give the same bits.
 *
 *   bias_gu    optional bf16 [E, N_gu] (16-byte aligned), added to the gate_up result in bf16 before the
 *              activation; fused launch only (GNF4B_EUNSUPPORTED otherwise)
 *   workspace  at least gnf4b_ffn_workspace_bytes(...) bytes, 256-byte aligned, zero-filled once before its first
 *              use (the kernels leave it as they need it); holds the intermediates and the group counters of the
 *              fused launch.  Calls that overlap on the GPU need separate workspaces.
 * Every device-side wait of the fused launch is bounded: on expiry GNF4B_ST_TIMEOUT is raised and the results are
 * void, nothing hangs.  GNF4B_ACT_GPT_OSS_GLU needs MXFP4 stacks on the fused path. */
int gnf4b_ffn_grouped(int fmt, int act, const void* x, int x_dtype, int64_t T,
                      const uint8_t* W_gu, int64_t wgu_stride_e, int64_t wgu_stride_n,
                      const void* S_gu, int64_t sgu_stride_e, int64_t sgu_stride_n,
                      const uint8_t* W_dn, int64_t wdn_stride_e, int64_t wdn_stride_n,
                      const void* S_dn, int64_t sdn_stride_e, int64_t sdn_stride_n, int s_dtype,
                      const void* bias_gu, const int32_t* group_offsets, const int32_t* expert_ids, int32_t G, int32_t E,
                      int64_t N_gu, int64_t K_gu, int64_t N_dn, int32_t max_rows, void* out, void* workspace,
                      size_t workspace_bytes, int32_t* status_word, uint32_t flags, void* cuda_stream);
size_t gnf4b_ffn_workspace_bytes(int fmt, int64_t T, int32_t G, int64_t N_gu, int64_t K_gu, int64_t N_dn,
                                 int32_t max_rows, uint32_t flags);

/* Scratch gnf4b_gemm_grouped needs for the same arguments (0 when none).  Replaces the
 * `ws = torch.empty(sk, T, N)` split-K buffer of kernel/nf4_grouped.py:784. */
size_t gnf4b_workspace_bytes(int fmt, int op, int64_t T, int32_t G, int64_t N, int64_t K,
                             int32_t max_rows, uint32_t flags);

/* The split-K factor the planner picks (or the forced one in `flags`), so a caller can
 * mirror _decode_plan (kernel/nf4_grouped.py:609-632) without launching. */
int gnf4b_plan_split_k(int fmt, int op, int64_t T, int32_t G, int64_t N, int64_t K,
                       int32_t max_rows, uint32_t flags);

/* sizes[G] (device int32) -> group_offsets[G+1] (device int32), one small kernel, no
 * host read.  Replaces the host loop of build_group_tiles (kernel/nf4_grouped.py:334-362)
 * when the group sizes live on the device. */
int gnf4b_build_offsets(const int32_t* sizes, int32_t G, int32_t* group_offsets,
                        void* cuda_stream);

/* Copy n int32 from (pinned) host memory to device memory on the stream, asynchronously:
 * one cudaMemcpyAsync.  This is how the small group tables travel; it replaces the
 * pageable / pinned-arena transfers of to_device_i32 (kernel/nf4_grouped.py:229-331). */
int gnf4b_upload_i32(const int32_t* host_src, int32_t* device_dst, int64_t n, void* cuda_stream);

/* Element decode of a whole stack with the SAME device decode routines the GEMM kernels
 * use: out_f32 [E, N, K] contiguous.  Counterpart of dequant_ref
 * (kernel/nf4_grouped.py:910-929) and dequant_mxfp4 (kernel/mxfp4_pack_ref.py:46-70);
 * exists so decode can be compared bit for bit. */
int gnf4b_dequant(int fmt,
                  const uint8_t* W, int64_t w_stride_e, int64_t w_stride_n,
                  const void* S, int s_dtype, int64_t s_stride_e, int64_t s_stride_n,
                  int32_t E, int64_t N, int64_t K, float* out_f32, void* cuda_stream);

/* Expert-parallel layer helpers.  The reference is single-GPU and has no counterpart; its offload
 * decode applies the same activation on the host side (bench/phase3/offload_decode_235b.py:232-233).
 *
 * gnf4b_silu_glu: gate_up [rows, 2h] bf16 -> out [rows, h] bf16 = silu(gate) * up, gate = first half
 * of each row, fp32 math, one rounding.
 *
 * gnf4b_combine_rows: out[m, :] (bf16 [M, H]) = sum_j weights[m, j] * rows[pos[m, j], :] over the k
 * routed copies of token m, j in order, fp32, multiply and add rounded separately: deterministic, and
 * equal bit for bit to the same loop written with tensor operations.  rows is bf16 [P, H]; a position
 * outside [0, P) is skipped and flagged GNF4B_ST_BAD_OFFSETS in the status word. */
int gnf4b_silu_glu(const void* gate_up, int64_t rows, int64_t h, void* out, void* cuda_stream);
/* The activation of gpt-oss between its expert GEMMs (kernel/mxfp4_pipelined.py:453-461): gate_up [rows, 2h] bf16 with
 * gate and up INTERLEAVED in the columns -> out [rows, h] bf16, every step rounded to bf16 as the reference's tensor
 * operations do.  bias (optional, bf16 [E, 2h]) is added first, row r taking bias[row_expert[r]]. */
int gnf4b_glu_gpt_oss(const void* gate_up, int64_t rows, int64_t h, const void* bias, const int32_t* row_expert,
                      void* out, void* cuda_stream);
int gnf4b_combine_rows(const void* rows, int64_t P, const int64_t* pos, const float* weights, int32_t k,
                       int64_t M, int64_t H, void* out, int32_t* status_word, void* cuda_stream);

/* Router selection on the device: logits fp32 [T, E] -> idx int64 [T, k] (the k largest, descending, ties to
 * the lower expert index) and weights fp32 [T, k] (mode 0: softmax over all E, norm != 0 renormalises over the
 * k; mode 1: softmax over the k selected).  The rule of the reference's CPU router
 * (gnf4_native/cpu_kernels.c:1408-1471); k <= 32. */
int gnf4b_route_topk(const float* logits, int64_t T, int32_t E, int32_t k, int32_t mode, int32_t norm, int64_t* idx,
                     float* weights, void* cuda_stream);

/* Fixed-capacity exchange of a small batch (P = tokens * top_k <= 1024 pairs, n_experts <= 1024), no host
 * read anywhere (expert-parallel layer; no reference counterpart).
 *
 * gnf4b_ep_plan, one CTA: idx[P] (int64 global expert ids, pair p = token p / k) -> counts[n_experts]
 * (int32 pairs per expert), slot[P] (int64 row of pair p in the send buffer: rank d = expert / e_local owns
 * rows [d * cap, (d + 1) * cap), ordered by local expert, pairs of one expert in pair order; -1 and
 * GNF4B_ST_BAD_EXPERT for an id outside [0, n_experts)), and the copy of the pairs' hidden rows (bf16
 * [tokens, H]) into send (bf16 [world * cap, H]).  cap >= the pairs any one rank can receive (cap = P is always
 * enough); a pair that does not fit its rank's cap rows gets slot -1, is not sent, and GNF4B_ST_BAD_OFFSETS is raised.
 *
 * gnf4b_ep_offsets: recv_counts[world, e_local] -> offsets[world * (e_local + 1) + 1] of the received buffer:
 * per source rank its e_local expert blocks, then the unused capacity as one group (to be given
 * GNF4B_PAD_EXPERT). */
int gnf4b_ep_plan(const int64_t* idx, int32_t P, int32_t k, int32_t n_experts, int32_t e_local, int32_t cap,
                  const void* hidden, int64_t H, int32_t* counts, int64_t* slot, void* send, int32_t* status_word,
                  void* cuda_stream);
int gnf4b_ep_offsets(const int32_t* recv_counts, int32_t world, int32_t e_local, int32_t cap, int32_t* offsets,
                     int32_t* status_word, void* cuda_stream);

/* Routing plan of a LARGE batch (any P up to 2^26 pairs): the stable sort of the pairs by (half, global expert id) as
 * a counting sort over several CTAs -- the order of a stable argsort of those keys -- and the gather of the pairs'
 * hidden rows into it.  half = 1 for experts whose local index (id % e_local) is >= cut (cut = e_local: one half);
 * with two halves every rank's lower experts come first, which lets a caller exchange and multiply them while the
 * upper half is still in flight.  Outputs: counts[n_experts] (int32 pairs per expert), pos[P] (int64 position of
 * pair p in the sorted order), send (bf16 [P, H]: send[pos[p]] = hidden[p / k]).  scratch: device memory of
 * gnf4b_ep_plan_large_scratch_bytes(P, n_experts) bytes, any content.  An id outside [0, n_experts) is flagged
 * GNF4B_ST_BAD_EXPERT and placed behind all valid pairs. */
size_t gnf4b_ep_plan_large_scratch_bytes(int64_t P, int32_t n_experts);
int gnf4b_ep_plan_large(const int64_t* idx, int64_t P, int32_t k, int32_t n_experts, int32_t e_local, int32_t cut,
                        const void* hidden, int64_t H, int32_t* counts, int64_t* pos, void* send, void* scratch,
                        size_t scratch_bytes, int32_t* status_word, void* cuda_stream);

/* Large-batch exchange without a collective library: up to GNF4B_EP_MAX_WORLD blocks of rows (src[b] -> dst[b], bytes[b]
 * a multiple of 16, dst typically a peer's symmetric buffer) copied by all SMs with plain 16-byte stores; when the last
 * CTA is through, behind a system-scope fence, flags[b] (this rank's flag word in peer b's buffer; may be null) is set
 * to `step`.  The blocks are taken 64 KiB at a time round by round, starting each round at block first_block (pass the
 * rank: a rank then writes to all peers at once and no two ranks start on the same peer).  done_counter: a device int32
 * of this rank that is zero before the first call (left at zero).  The
 * receiver queues gnf4b_ep_wait_flags(its flag words, world, step) before the kernels that read the rows: a bounded
 * wait (timeout_ms; GNF4B_ST_TIMEOUT in the status word on expiry) until every flag has reached `step` (flags only
 * grow).  The caller sees to it that a block's destination is free: in ep_moe a rank pushes step n + 1 only after its
 * combine of step n has heard from every rank. */
int gnf4b_ep_push_blocks(int32_t n, const void* const* src, void* const* dst, const int64_t* bytes, int32_t* const* flags,
                         int32_t step, int32_t first_block, int32_t* done_counter, void* cuda_stream);
int gnf4b_ep_wait_flags(const int32_t* flags, int32_t world, int32_t step, int32_t timeout_ms, int32_t* status_word,
                        void* cuda_stream);

/* The same small-batch exchange without a collective library (expert-parallel layer; no reference counterpart):
 * each rank owns ONE exchange buffer of gnf4b_ep_peer_layout(...)[0] bytes that every other rank of the node can
 * address (peer access / symmetric memory); ctx.peers[r] is rank r's buffer as THIS process addresses it, 256-byte
 * aligned, zeroed once before the first step with a barrier of the ranks after the zeroing.  Rows travel as plain
 * stores to the peer pointer, every 8 bytes carrying 4 bytes of row and the 4-byte number of the step; a reader that
 * finds the number it expects has the payload beside it, so there is no fence, no flag and no multicast.  Per layer,
 * on every rank, two launches around the GEMMs on one stream (each may be replayed from a captured graph: the step
 * numbers live in the buffer).  Each launch first sends and then receives, so no rank waits before it has sent:
 *
 *   gnf4b_ep_peer_dispatch  SENDS: the plan of gnf4b_ep_plan (slot[P] as there); rows and per-expert counts written
 *                           into the destinations' buffers.  RECEIVES: waits for all sources' counts and for the rows
 *                           they announce, unpacks the rows EXPERT-MAJOR (local experts ascending; inside an expert
 *                           sources in rank order, a source's rows in the order sent) into the row matrix bf16
 *                           [world * cap, H] at byte layout[1] of the own buffer, and writes the group tables of the
 *                           GEMMs over that matrix:
 *                             one_row_groups = 0: offsets[e_local + 1] (the groups are the local experts 0 .. e_local-1)
 *                             one_row_groups = 1: every row its own group, offsets[world * cap + 1] (offsets[g] =
 *                               min(g, rows)) and expert_ids[world * cap] (the row's expert, GNF4B_PAD_EXPERT beyond
 *                               the rows): few rows, the one-row kernels (max_rows = 1) apply.
 *   (the grouped GEMMs and the activation on that matrix, result y bf16 [world * cap, H] in the same row order)
 *   gnf4b_ep_peer_combine   SENDS: every result row of y back to its source's buffer, and to every rank the word
 *                           that this rank is through with what it received.  RECEIVES: waits for that word from
 *                           every rank and for the rows it expects, then out[m] = sum_j weights[m, j] *
 *                           returned[slot[m, j]] with the arithmetic of gnf4b_combine_rows.
 *
 * All ranks call with the same cap (<= cap_max, world * cap <= 1024) and H (% 8 == 0).  Every wait is bounded (2 s):
 * when it runs out GNF4B_ST_TIMEOUT is raised in the status word and the kernel goes on with what is there.  One set
 * of row slots is enough because the steps interlock: a rank's next dispatch follows its combine, which has heard
 * from every rank's combine, which follows that rank's dispatch. */
#define GNF4B_EP_MAX_WORLD 16
typedef struct gnf4b_ep_peer_ctx {
    int32_t world, rank, e_local, cap_max;
    int64_t H;
    void* peers[GNF4B_EP_MAX_WORLD];
} gnf4b_ep_peer_ctx;
/* out3 = {bytes of one rank's buffer, byte offset of the row matrix, byte offset of the returned rows' slots} */
int gnf4b_ep_peer_layout(int32_t world, int32_t e_local, int32_t cap_max, int64_t H, int64_t* out3);
int gnf4b_ep_peer_dispatch(const gnf4b_ep_peer_ctx* ctx, const int64_t* idx, int32_t P, int32_t k, int32_t n_experts,
                           int32_t cap, const void* hidden, int64_t* slot, int32_t one_row_groups, int32_t* offsets,
                           int32_t* expert_ids, int32_t* status_word, void* cuda_stream);
int gnf4b_ep_peer_combine(const gnf4b_ep_peer_ctx* ctx, int32_t cap, const void* y, const int64_t* slot,
                          const float* weights, int32_t k, int64_t M, void* out, int32_t* status_word, void* cuda_stream);

/* Residency feeders: an expert's packed row-block into a device slot, selected on the device (no host read, nothing
 * synchronises).  Format-agnostic byte movers; rows, offsets and lengths are multiples of 8 bytes (GNF4B_ESHAPE
 * otherwise).  A slot that already holds the wanted row is skipped without touching the source.  The source may be
 * device memory or pinned host memory that the GPU addresses directly.
 *
 * gnf4b_gather_rows_by_id   dst[slot] <- src[ids[slot]] (rows of row_bytes), skipped where have_ids[slot] == ids[slot]
 *                           (have_ids optional).  The reference's gather_expert_rows (kernel/host_gather.py:73-95).
 *                           An id outside [0, n_rows_src) is skipped and flagged GNF4B_ST_BAD_EXPERT (n_rows_src = 0:
 *                           not checked above).
 * gnf4b_gather_rows_addr    dst[slot] <- the row at absolute address want_addr[slot], skipped where have_addr[slot] ==
 *                           want_addr[slot] (optional) or the address is 0.  The reference's _gather_rows_addr
 *                           (kernel/mxfp4_pipelined.py:48-60).  With pieces (device int64 [n_pieces, 3] = source
 *                           offset, slot offset, length in bytes; max_piece_bytes = the longest) the row's segments
 *                           land in a different order: _gather_rows_perm (kernel/mxfp4_residency.py:117-134). */
int gnf4b_gather_rows_by_id(void* dst, int64_t row_bytes, int32_t n_slots, const void* src, int32_t n_rows_src,
                            const int32_t* ids, const int32_t* have_ids, int32_t* status_word, void* cuda_stream);
int gnf4b_gather_rows_addr(void* dst, int64_t row_bytes, int32_t n_slots, const int64_t* want_addr,
                           const int64_t* have_addr, const int64_t* pieces, int32_t n_pieces, int64_t max_piece_bytes,
                           void* cuda_stream);

/* Device properties this library plans with (SM count, opt-in shared memory). */
int gnf4b_device_info(int32_t* sm_count, int32_t* smem_optin_bytes);

#ifdef __cplusplus
}
#endif
#endif /* GNF4B_H_ */
