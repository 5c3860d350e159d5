/* C ABI of the B200 (sm_100a) quantized-decode library: GGUF block-quantized
 * GEMV / batched GEMM with per-32 int8 activations, MoE routing and the packed
 * expert feed-forward.
 *
 * This is the boundary a binding of the reference library
 * (cwpearson/dnn-for-kokkos) would call from inside its own operator templates;
 * each entry point names the reference operator it stands in for (paths are
 * relative to the reference project root). include/KokkosDNN_B200.hpp holds the
 * C++ layer that keeps the reference's Kokkos::View signatures on top of it.
 *
 * Conventions
 *   - every pointer is a device pointer valid on the current CUDA device unless
 *     a parameter comment says "host";
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *     stream, which is what Kokkos::Cuda().cuda_stream() callers pass);
 *   - calls are asynchronous: they enqueue kernels on `stream` and return;
 *   - nothing here allocates device memory; scratch and workspaces are
 *     caller-owned, sized by the *_bytes queries;
 *   - return value: KDNN_OK (0) launched; KDNN_DECLINED (1) the fast path does
 *     not cover this call and NOTHING was launched (the reference convention of
 *     src/KokkosDNN_GGUFGemvInt8.hpp:708-710: the caller runs its own portable
 *     path); negative = error, nothing launched, kdnn_b200_last_error() has text.
 *   - weight payloads are ggml blocks, unchanged: Q8_0 (34 B / 32), Q4_K
 *     (144 B / 256), Q6_K (210 B / 256), rows contiguous with stride
 *     row_bytes = cols / block_len * block_bytes.
 */
#ifndef KDNN_B200_H
#define KDNN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  KDNN_OK              = 0,
  KDNN_DECLINED        = 1,
  KDNN_ERR_INVALID     = -1, /* maps to std::invalid_argument in the C++ layer */
  KDNN_ERR_UNSUPPORTED = -2,
  KDNN_ERR_CUDA        = -3,
  KDNN_ERR_DEVICE_WAIT = -4  /* a bounded device-side wait gave up */
};

/* ggml type ids (src/KokkosDNN_GGUF.hpp:68-87). */
enum { KDNN_GGML_Q8_0 = 8, KDNN_GGML_Q4_K = 12, KDNN_GGML_Q5_K = 13, KDNN_GGML_Q6_K = 14 };

/* Scalar of activations / outputs (src/KokkosDNN_Types.hpp:16-18). */
enum { KDNN_F32 = 0, KDNN_BF16 = 1 };

/* Text of the last error on this host thread ("" if none). */
const char* kdnn_b200_last_error(void);

/* Reads and clears the device-side status word (0 = no bounded wait gave up).
 * Synchronizes the device. */
int kdnn_b200_device_status(void);

/* ---- GEMV -------------------------------------------------------------- */

/* Bytes of activation staging for a K-element row; 0 when K % 32 != 0.
 * Stands in for Gguf::quant_gemv_int8_scratch_bytes, src/KokkosDNN_GGUF.hpp:2496-2499.
 * Layout written: int8 xq[K], then at align16(K) one {float d; int32 sum_lo;
 * int32 sum_hi; int32 pad} per 32 elements (src/KokkosDNN_GGUFGemvInt8.hpp:108-129). */
size_t kdnn_b200_gemv_scratch_bytes(size_t K);

/* 1 when kdnn_b200_quant_gemv takes the int8 path for this weight type, K and
 * Scalar. Stands in for Gguf::quant_gemv_int8_supported, src/KokkosDNN_GGUF.hpp:2522-2529. */
int kdnn_b200_gemv_supported(uint32_t ggml_type, size_t K, int scalar);

/* y[rows] = W[rows, cols] . x[cols], int8 path: x is quantized per 32 elements
 * (d = amax/127, q = rint(x * (127/amax)) clamped to +-127, half sums) inside
 * the kernel's prologue, the integer dots run on dp4a, rescale in fp32.
 * Stands in for Gguf::quant_gemv(handle, x, w, y, act_scratch),
 * src/KokkosDNN_GGUF.hpp:2531-2551 -> Impl::GgufMvq::launch_quant_gemv_int8,
 * src/KokkosDNN_GGUFGemvInt8.hpp:711-777 (both of its launches in one kernel).
 * The staging bytes are also written to act_scratch, as the reference leaves them.
 *   x_scalar / y_scalar: KDNN_F32 or KDNN_BF16 (the reference uses one Scalar for
 *     both; y_scalar = KDNN_F32 with bf16 x gives the row sums before the cast).
 * Declines (returns KDNN_DECLINED) exactly where the reference's launcher does:
 * null w or scratch, K not block aligned, rows == 0 or > INT_MAX, scratch too
 * small or not 16-byte aligned, odd w, Q4_K w not 16-byte aligned. */
int kdnn_b200_quant_gemv(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                         const void* x, int x_scalar, void* y, int y_scalar,
                         void* act_scratch, size_t act_scratch_bytes, void* stream);

/* Optional tuning of one GEMV call; all zero = the library's own choice. Stands in for
 * Impl::GgufMvq::Int8Layout, src/KokkosDNN_GGUFGemvInt8.hpp:604-608 (rows_per_group keeps its meaning:
 * weight rows that share one pass over the activation window; the other fields name this library's
 * kernels instead of the reference's threads_per_row / groups). Results do not depend on it beyond
 * fp32 summation order. */
typedef struct {
  int kernel;         /* 0 auto; 1 activation window in registers; 2 window in shared memory;
                         3 item mapping with the window in shared memory; 4 plain loads (any alignment) */
  int rows_per_group; /* 0 auto; 1 or 2 */
  int stages;         /* 0 auto; 2..4 ring stages per warp */
  int early_stages;   /* 0 auto; ring stages requested before the activation row is quantized */
  int warps;          /* 0 auto; warps per CTA */
  int no_pdl;         /* 1: launch without programmatic stream serialization */
} kdnn_b200_gemv_layout;

/* kdnn_b200_quant_gemv with a tuning struct (NULL = defaults). */
int kdnn_b200_quant_gemv_ex(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                            const void* x, int x_scalar, void* y, int y_scalar,
                            void* act_scratch, size_t act_scratch_bytes,
                            const kdnn_b200_gemv_layout* layout, void* stream);

/* Launch chaining and the weights. Every kernel of this library is launched as a programmatic dependent of the
 * kernel before it on the stream and requests its first PACKED WEIGHT bytes before it waits for that kernel
 * (activations, routing and workspaces are only touched after the wait). So packed weights (w, the expert
 * payloads) must be complete and visible before the PREVIOUS kernel on the stream starts: weights that were
 * uploaded, repacked or dequantized on the same stream need a stream / event synchronisation before the first
 * call that reads them (the Python loaders do that), or chaining switched off around that call.
 * kdnn_b200_launch_chaining(0 / 1) switches it for the whole process and returns the previous setting;
 * a negative argument only queries. Results do not depend on it. */
int kdnn_b200_launch_chaining(int on);

/* n matrices of ONE format and shape against the SAME activation row: y[i] = W[i] . x, i < n. A decoder calls the
 * reference's quant_gemv once per projection with the same normed row (wgate and wup of the feed-forward,
 * models/glimmer/KokkosDNN_GlimmerModel.hpp:650-653; wk and wv, :523-526); this entry point takes those calls
 * together, and for Q4_K rows of up to 4096 elements runs up to four matrices per launch, so the ramp and the
 * tail of a launch that streams only tens of MB are paid once. Other formats and longer rows run as n launches.
 * w and y are HOST arrays of n device pointers. Results equal n calls of kdnn_b200_quant_gemv bit for bit.
 * Declines as kdnn_b200_quant_gemv does, for any of the matrices, before anything is launched. */
int kdnn_b200_quant_gemv_multi(uint32_t ggml_type, size_t n, const void* const* w, size_t rows, size_t cols,
                               const void* x, int x_scalar, void* const* y, int y_scalar, void* act_scratch,
                               size_t act_scratch_bytes, const kdnn_b200_gemv_layout* layout, void* stream);

/* The same GEMV for callers that have no scratch buffer to give and may not create one: a
 * host runtime that reserved the whole device up front and forbids cudaMalloc in its
 * plug-ins, or a decode loop that is not allowed to touch the allocator because an
 * allocation can stall every stream of the device. The activation staging lives in a
 * fixed 48 KB array inside the library's device image instead (every GPU that loads the
 * library holds it until the process exits), so the limit is cols <= 32768; larger K is
 * rejected with KDNN_ERR_INVALID and a message that names the limit. The call allocates
 * nothing (no cudaMalloc / cudaFree, no allocating library routine). Its first call on a
 * device looks up the array's device address (with that device current) and caches it;
 * make that first call outside any stream capture. All calls on a device share the one
 * array: it keeps the previous call's staging (every byte the kernels read is rewritten
 * first, nothing has to start at zero), and two calls that overlap on the GPU -- different
 * streams, or concurrent host threads -- race on it; serialise them or use
 * kdnn_b200_quant_gemv. Results are identical to kdnn_b200_quant_gemv.
 * This entry point has no counterpart in the reference, whose operator always takes the
 * caller's act_scratch view. */
int kdnn_b200_quant_gemv_noalloc(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                                 const void* x, int x_scalar, void* y, int y_scalar, void* stream);
/* The same entry point with the tuning struct of kdnn_b200_quant_gemv_ex (NULL = defaults); x and y must
 * have unit stride, as everywhere. No counterpart in the reference either. */
int kdnn_b200_quant_gemv_noalloc_ex(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                                    const void* x, int x_scalar, void* y, int y_scalar,
                                    const kdnn_b200_gemv_layout* layout, void* stream);

/* kdnn_b200_quant_gemv for a host that keeps activations and results in its own (ideally page-locked)
 * memory: one call enqueues the copy of x_host[cols] to x_dev, the GEMV, and the copy of y_dev[rows] to
 * y_host on `stream`, and returns without waiting; y_host is valid once the stream has been synchronised.
 * x_dev, y_dev and act_scratch are the caller's device buffers (nothing is allocated). A declined or
 * failed call has enqueued nothing. When the host buffers are page-locked (or registered) and 16-byte
 * aligned the two copies are small kernels over the mapped host pointers, chained with the GEMV like every
 * kernel of the library (the copy engine's hand-offs cost more than these kernels do); pageable buffers,
 * or every buffer after kdnn_b200_host_copy_by_kernel(0), take cudaMemcpyAsync. In the reference this is the host's
 * deep_copy, quant_gemv, deep_copy
 * sequence around src/KokkosDNN_GGUF.hpp:2531-2551 folded into one call; same decline list and results. */
int kdnn_b200_quant_gemv_host(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                              const void* x_host, int x_scalar, void* y_host, int y_scalar, void* x_dev,
                              void* y_dev, void* act_scratch, size_t act_scratch_bytes, void* stream);
/* 1 (default): page-locked host buffers of kdnn_b200_quant_gemv_host are moved by kernels; 0: always by the copy
 * engine. Returns the previous setting; a negative argument only queries. */
int kdnn_b200_host_copy_by_kernel(int on);

/* Stage 1 alone: quantize one activation row into `scratch` (layout above).
 * Stands in for Impl::GgufMvq::QuantizeActQ8Functor, src/KokkosDNN_GGUFGemvInt8.hpp:198-239. */
int kdnn_b200_quantize_act_q8(const void* x, int x_scalar, size_t K, void* scratch,
                              size_t scratch_bytes, void* stream);

/* Parity probe: the integer dots of every decode unit (32 weights of one row)
 * against an already staged activation row, exactly the integers the reference
 * multiplies by its fp32 scales in Impl::GgufMvq::gemv_int8_unit_dot_win,
 * src/KokkosDNN_GGUFGemvInt8.hpp:359-466:
 *   Q4_K: {dotA, dotB}   Q6_K: {dotA - 32*sum0, dotB - 32*sum1}   Q8_0: {dot, 0}
 * out: int32[rows * (cols/32) * 2]. */
int kdnn_b200_unit_dots(uint32_t ggml_type, const void* w, size_t rows, size_t cols,
                        const void* staged_scratch, int32_t* out, void* stream);

/* ---- batched GEMV / skinny GEMM ------------------------------------------ */

/* Workspace bytes for kdnn_b200_quant_gemm with M activation rows of K elements. */
size_t kdnn_b200_gemm_workspace_bytes(size_t M, size_t K);

/* Y[M, N] = X[M, K] . W[N, K]^T with packed W, every activation row quantized per
 * 32 elements as in the GEMV, so row m of Y equals kdnn_b200_quant_gemv on row m.
 * Stands in for Gguf::quant_gemm, src/KokkosDNN_GGUF.hpp:2564-2593 (which is the
 * fp path; the int8 numerics follow src/KokkosDNN_GGUFGemvInt8.hpp per row).
 *   ldx, ldy: row pitches in elements. */
int kdnn_b200_quant_gemm(uint32_t ggml_type, const void* w, size_t N, size_t K,
                         const void* X, size_t ldx, size_t M, int x_scalar,
                         void* Y, size_t ldy, int y_scalar,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Parity probe of the batched path: kdnn_b200_quant_gemm on the tcgen05 tile kernel that additionally
 * stores the raw int32 sub-block dots the tensor cores produced, dots[m][n][K/32] (Q4_K: the integer
 * sum over 32 elements of nibble * xq, the factor the reference multiplies by d*sc*dx,
 * src/KokkosDNN_GGUFGemvInt8.hpp:359-388). KDNN_DECLINED when the tcgen05 kernel does not serve the call. */
int kdnn_b200_quant_gemm_dots(uint32_t ggml_type, const void* w, size_t N, size_t K,
                              const void* X, size_t ldx, size_t M, int x_scalar,
                              void* Y, size_t ldy, int y_scalar, int32_t* dots,
                              void* workspace, size_t workspace_bytes, void* stream);

/* Which kernel the batched Q4_K calls (quant_gemm, moe_ffn, moe_block) use from now on, process-wide:
 * 3 = by measured crossover (the default: quant_gemm runs the GEMV kernel per row up to 3 activation rows,
 * the tcgen05 kernel up to 8, the mma.sync kernel beyond; the MoE feed-forward runs the mma.sync kernel),
 * 2 = tcgen05.mma + TMEM fed by tensor-map TMA wherever it applies, 1 = mma.sync m16n8k32, 0 = the
 * CUDA-core dp4a kernel that serves every other format. Returns the previous kind; kind < 0 only queries.
 * A tuning knob in the sense of Int8Layout (src/KokkosDNN_GGUFGemvInt8.hpp:604-608); results agree
 * within fp32 summation order. */
int kdnn_b200_tile_kind(int kind);

/* ---- MoE ------------------------------------------------------------------ */

/* Per-token top-k expert selection and combination weights.
 * Stands in for KokkosDNN::moe_route (sigmoid = 0), src/KokkosDNN_MoE.hpp:240-263,
 * and KokkosDNN::moe_route_sigmoid (sigmoid = 1), :280-304. Greedy selection with
 * strict '>' (ties keep the lower expert id); weights recomputed from the logits
 * at the selected ids (:84-147).
 *   logits [T, E] Scalar, row pitch ld (elements); bias [E] Scalar or NULL;
 *   top_idx [T, top_k] int32; top_w [T, top_k] float. */
int kdnn_b200_moe_route(const void* logits, size_t ld, size_t T, size_t E, int scalar,
                        const void* bias, int top_k, int norm_topk, float routed_scale,
                        int sigmoid, int32_t* top_idx, float* top_w, void* stream);

/* One packed expert matrix kind (gate, up or down): device array of n_experts
 * payload pointers plus the shape every entry shares.
 * Mirrors Gguf::QuantWeightTable, src/KokkosDNN_GGUF.hpp:2020-2029. */
typedef struct {
  const uintptr_t* base; /* device array [n_experts] of payload addresses */
  uint32_t ggml_type;
  size_t rows, cols, row_bytes;
  size_t n_experts;
  const void* tma;       /* device array [n_experts] of 128-byte TMA descriptors written by
                            kdnn_b200_weight_table_tma_encode, or NULL (the tcgen05 tile kernel then
                            leaves the call to the mma.sync kernel) */
} kdnn_b200_weight_table;

/* Bytes of the descriptor array of a table with n_experts entries (128 each). */
size_t kdnn_b200_weight_table_tma_bytes(size_t n_experts);

/* Fills host_out[n_experts * 128] with one TMA descriptor per expert matrix (host_base: the payload
 * addresses on the HOST, i.e. what make_quant_weight_table copies to the device,
 * src/KokkosDNN_GGUF.hpp:2031-2053). The caller copies host_out to 128-byte aligned device memory and
 * points `tma` at it; payloads must not move afterwards (they never do after load,
 * models/lfm2_5/KokkosDNN_LFM25Model.hpp:557-560). Only Q4_K tables have a tensor-core kernel:
 * KDNN_DECLINED for other types (leave `tma` NULL). Pure host work, no launch, no allocation. */
int kdnn_b200_weight_table_tma_encode(const uintptr_t* host_base, uint32_t ggml_type, size_t rows, size_t cols,
                                      size_t n_experts, void* host_out);

/* Workspace bytes for kdnn_b200_moe_ffn with T tokens, S slots per token. */
size_t kdnn_b200_moe_workspace_bytes(size_t T, size_t S, size_t H, size_t F, size_t n_experts);

/* Expert feed-forward for T tokens with int8 activations:
 *   per (token t, slot s), e = idx[t,s] (slots with e outside [0, n_experts) or
 *   w == 0 contribute nothing): act = Scalar(silu(gate_e x_t) * (up_e x_t)),
 *   Y[t,:] = Scalar(sum_s w[t,s] * (down_e act)), slots ascending, fp32.
 * T == 1 stands in for Gguf::quant_moe_decode, src/KokkosDNN_GGUF.hpp:2335-2391;
 * T > 1 for the per-expert gather / dequant / gemm / swiglu / gemm / scatter loop
 * of LFM2.5's moe_forward_sparse, models/lfm2_5/KokkosDNN_LFM25Model.hpp:441-547.
 *   X [T, H] Scalar pitch ldx; idx [T, S] int32; wts [T, S] float;
 *   Y [T, H] y_scalar pitch ldy (assigned, not accumulated);
 *   expert_first / expert_count: only experts in [first, first+count) are
 *   computed here (expert-parallel shard); pass 0, n_experts for all. */
int kdnn_b200_moe_ffn(const void* X, size_t ldx, size_t T, int x_scalar,
                      const kdnn_b200_weight_table* gate, const kdnn_b200_weight_table* up,
                      const kdnn_b200_weight_table* down, const int32_t* idx, const float* wts,
                      size_t S, void* Y, size_t ldy, int y_scalar,
                      size_t expert_first, size_t expert_count,
                      void* workspace, size_t workspace_bytes, void* stream);

/* ---- the MoE block in four launches, single GPU or expert-parallel --------------------------------- */

/* Expert-parallel exchange over peer memory (NVLink): every rank owns one region of
 * kdnn_b200_moe_exchange_bytes() that ALL ranks can address (cudaMalloc + cudaIpc handles, or any other
 * peer-mapped allocation; zero it once before the first call). `regions[r]` is rank r's region as seen from
 * THIS process; regions[rank] is the local one. Every rank makes the same sequence of block calls with the
 * same tokens_local, world, top_k and hidden size. No counterpart in the reference, which is single-device
 * (there is no collective anywhere in it); the partition rule is expert e on rank e / (E / world). */
typedef struct {
  int rank, world;            /* world <= 8 */
  void* const* regions;       /* host array [world] of device addresses */
  unsigned long long wait_ns; /* bound of every device-side wait for a peer; 0 = 2 s */
} kdnn_b200_moe_exchange;

size_t kdnn_b200_moe_exchange_bytes(size_t tokens_local, size_t world, size_t top_k, size_t H);

/* Workspace bytes of kdnn_b200_moe_block (256-byte aligned, zeroed once before the first call;
 * with_region != 0 includes the exchange region of a single-GPU call). */
size_t kdnn_b200_moe_block_workspace_bytes(size_t tokens_local, size_t world, size_t top_k, size_t H, size_t F,
                                           size_t n_experts, int with_region);

/* One MoE block for this rank's tokens_local tokens:
 *   logits = Scalar(x . router_w^T)  (the caller's gemm, models/lfm2_5/KokkosDNN_LFM25Model.hpp:796)
 *   -> moe_route / moe_route_sigmoid (src/KokkosDNN_MoE.hpp:240-304)
 *   -> the expert feed-forward with int8 activations on this rank's experts [expert_first, +expert_count)
 *      for the routed slots of ALL ranks' tokens (kdnn_b200_moe_ffn's numerics)
 *   -> y = sum over the slots (slot order, fp32) on the token's owner
 *   -> optionally h_out = Scalar(float(resid) + y) (:812-816) and xn_out = rmsnorm_noscale(h_out)
 *      (src/KokkosDNN_RMSNorm.hpp:347-361, the next block's :770).
 * Four kernel launches: router + routing + row quantizer + slot runs, gate/up tiles, down tiles, combine.
 * With `ex` != NULL rank r owns tokens [r * tokens_local, (r + 1) * tokens_local) and experts
 * [r * E / world, (r + 1) * E / world) (expert_first / expert_count must say so, KDNN_ERR_INVALID otherwise):
 * the quantized token rows and routed ids travel to every rank inside the first kernel (plain peer stores, one
 * atomic add per routed slot on the expert owner's counter), the down kernel leaves its output rows in its own
 * rank's region and the token owner's combine kernel reads them from there (plain peer loads). Every wait for a
 * peer is bounded (KDNN_ERR_DEVICE_WAIT in kdnn_b200_device_status() when one gave up; the call never hangs).
 * The workspace carries the call's epoch counters: one workspace per stream, the same one for every call of a
 * sequence.
 *   x [tokens_local, H] Scalar; router_w [E, H] Scalar, 16-byte aligned rows; router_bias [E] or NULL;
 *   y [tokens_local, H] float or NULL; resid / h_out / xn_out [tokens_local, H] Scalar or NULL.
 * Q4_K tables only (KDNN_DECLINED otherwise: compose kdnn_b200_moe_route + kdnn_b200_moe_ffn instead). */
int kdnn_b200_moe_block(const void* x, size_t ldx, size_t tokens_local, int scalar,
                        const void* router_w, size_t ldr, const void* router_bias,
                        int top_k, int norm_topk, float routed_scale, int sigmoid,
                        const kdnn_b200_weight_table* gate, const kdnn_b200_weight_table* up,
                        const kdnn_b200_weight_table* down, size_t expert_first, size_t expert_count,
                        float* y, size_t ldy, const void* resid, size_t ldres, void* h_out, size_t ldh,
                        void* xn_out, size_t ldxn, float eps,
                        const kdnn_b200_moe_exchange* ex, void* workspace, size_t workspace_bytes, void* stream);

/* Copies the routing result of the last kdnn_b200_moe_block call out of the exchange region / workspace into
 * the caller's device buffers, on `stream`: idx_out [T, top_k] int32 (all ranks' tokens, token-major over the
 * ranks), wts_out [T, top_k] float (only the rows of THIS rank's tokens are meaningful: the weights do not travel). */
int kdnn_b200_moe_block_routing(const kdnn_b200_moe_exchange* ex, void* workspace, size_t tokens_local, size_t world,
                                size_t top_k, size_t H, size_t F, size_t n_experts, int32_t* idx_out, float* wts_out,
                                void* stream);

/* Peer-visible device memory for the exchange regions: cudaMalloc + cudaIpcGetMemHandle on the owner,
 * cudaIpcOpenMemHandle on the peers (handle = 64 opaque bytes to pass between the processes). These are
 * the only entry points of the library that allocate. */
int kdnn_b200_peer_alloc(size_t bytes, void** ptr, void* handle64);
int kdnn_b200_peer_open(const void* handle64, void** ptr);
int kdnn_b200_peer_close(void* ptr);
int kdnn_b200_peer_free(void* ptr);

/* out[t,:] = Scalar(r / sqrt(mean(r^2) + eps)), r = Scalar(float(h[t,:]) + y[t,:]): the residual add that
 * follows the MoE block (models/lfm2_5/KokkosDNN_LFM25Model.hpp:812-816) fused with the next block's
 * un-scaled RMS norm, KokkosDNN::rmsnorm_noscale, src/KokkosDNN_RMSNorm.hpp:347-361.
 *   h, out [T, H] Scalar (pitches ldh, ldo); y [T, H] float (pitch ldy), e.g. the fp32 output of
 *   kdnn_b200_moe_ffn. */
int kdnn_b200_residual_rmsnorm(const void* h, size_t ldh, const float* y, size_t ldy, void* out, size_t ldo,
                               size_t T, size_t H, float eps, int scalar, void* stream);

/* ---- the small MoE operators, for callers that keep the reference's per-expert loop ------------------
 * (models/lfm2_5/KokkosDNN_LFM25Model.hpp:441-547). Rows are contiguous, pitches in elements; argument
 * errors the reference throws for return KDNN_ERR_INVALID; zero extents return KDNN_OK without a launch. */

/* out[t, f] = Scalar(silu(float(gate[t, f])) * float(up[t, f])), fp32 arithmetic:
 * KokkosDNN::swiglu, src/KokkosDNN_SwiGLU.hpp:24-38 (silu :12-14). */
int kdnn_b200_swiglu(const void* gate, size_t ldg, const void* up, size_t ldu, void* out, size_t ldo, size_t T, size_t F,
                     int scalar, void* stream);

/* y[t, d] = Scalar(sum_k top_w[t, k] * float(expert_out[t, k, d])), k ascending, fp32:
 * KokkosDNN::moe_expert_weighted_sum, src/KokkosDNN_MoE.hpp:313-332. expert_out [T, K, D] contiguous. */
int kdnn_b200_moe_expert_weighted_sum(const void* expert_out, const float* top_w, void* y, size_t ldy, size_t T, size_t K,
                                      size_t D, int scalar, void* stream);

/* dst[n, :] = src[rows[n], :], 0 <= rows[n] < C (not checked on the device, as in the reference):
 * KokkosDNN::moe_gather_rows, src/KokkosDNN_MoE.hpp:337-351. */
int kdnn_b200_moe_gather_rows(const void* src, size_t lds, size_t C, const int32_t* rows, void* dst, size_t ldd, size_t N,
                              size_t D, int scalar, void* stream);

/* dst[rows[n], d] = Scalar(float(dst[rows[n], d]) + weights[n] * float(src[n, d])); `rows` must hold unique
 * entries (no atomics): KokkosDNN::moe_scatter_add_weighted, src/KokkosDNN_MoE.hpp:360-381. */
int kdnn_b200_moe_scatter_add_weighted(const void* src, size_t lds, const int32_t* rows, const float* weights, void* dst,
                                       size_t ldd, size_t C, size_t N, size_t D, int scalar, void* stream);

/* Measurement aid: streams [src, src + bytes) once with 128-bit read-only loads and discards the data
 * (`sink`: one device word). The read-only ceiling next to which the reference quotes its GEMV bandwidths
 * (benchmarks/Bench_GGUFGemv.cpp:65-81, benchmarks/Bench_MoeDecode.cpp:217-257). src 16-byte aligned. */
int kdnn_b200_read_probe(const void* src, size_t bytes, void* sink, void* stream);

/* Y[r, k] = Scalar(dequant(W[r, k])): replaces KokkosDNN::Gguf::dequant_to_dense,
 * src/KokkosDNN_GGUF.hpp:2839-2934 (block formulas :300-384). Types Q4_K, Q5_K, Q6_K, Q8_0; fp32 outputs are
 * bit-identical to the reference's (same association, no fused multiply-add), bf16 outputs are their
 * round-to-nearest-even.
 *   w [rows * row_bytes] packed rows; y [rows, cols] Scalar with pitch ldy (elements, >= cols).
 * KDNN_ERR_INVALID for an unknown type, cols that are not a whole number of blocks (256 for the K-quants,
 * 32 for Q8_0) or ldy < cols (the reference throws std::invalid_argument for those); zero extents return
 * KDNN_OK without a launch. */
int kdnn_b200_dequant_to_dense(uint32_t ggml_type, const void* w, size_t rows, size_t cols, void* y, size_t ldy,
                               int y_scalar, void* stream);

/* y[N] = Scalar(sum_k dequant(W[n,k]) * float(x[k])) with fp32 accumulation: replaces the staging-free
 * KokkosDNN::Gguf::quant_gemv(handle, x, w, y), src/KokkosDNN_GGUF.hpp:2394-2493 (the fp path a declined
 * int8 call falls back to). Types Q4_K, Q5_K, Q6_K, Q8_0. The weights are the reference's dequantized values
 * bit for bit; the order of the fp32 additions differs from its FMA chains, so results agree to fp32 rounding
 * of the sum, not bit for bit. Any payload alignment; x, y unit stride.
 * KDNN_ERR_INVALID for an unknown type or cols that are not a whole number of blocks (the reference's
 * quant_check); zero extents return KDNN_OK without a launch. */
int kdnn_b200_quant_gemv_fp(uint32_t ggml_type, const void* w, size_t rows, size_t cols, const void* x,
                            int x_scalar, void* y, int y_scalar, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KDNN_B200_H */
