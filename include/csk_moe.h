/* csk_moe.h -- C ABI of the B200 (sm_100a) mixture-of-experts layer.
 *
 * One opaque handle per MoE layer and device.  The handle owns the repacked
 * MXFP4 expert weights, the router weights and all scratch memory on that
 * device.  Every function returns 0 on success or a negative csk_status; no
 * C++ exception crosses this boundary and nothing here aborts the process.
 * csk_moe_last_error() gives the text of the last failure.
 *
 * Calls on one handle must be serialised by the caller; calls on different
 * handles may run concurrently from different host threads (the reference
 * drives each layer from its own scheduler thread, one frame in flight:
 * include/coalsack/nn/model_io_nodes.h:268-290, src/llm/llm_engine.cpp:904).
 *
 * "reference" below means the yoshou/coalsack source tree; paths are relative
 * to its root.  Tensor conventions are the reference's:
 *   hidden      [T, H] fp32 row-major   (the reference's [batch, seq, H], T = batch*seq)
 *   router_out  [T, k, 2] fp32          (expert id stored as a float, routing weight)
 *   MXFP4       row-major rows of cols/32 blocks of 17 bytes: one E8M0 scale
 *               byte, then 16 bytes of E2M1 codes; byte j holds element j in
 *               its low nibble and element j+16 in its high nibble
 *               (include/coalsack/tensor/dynamic_mx_tensor.h:19-44,
 *                include/coalsack/gguf/gguf_dequant.h:437-455).
 */
#ifndef CSK_MOE_H
#define CSK_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum csk_status {
  CSK_OK = 0,
  CSK_ERR_INVALID = -1,  /* bad argument, shape or state                         */
  CSK_ERR_CUDA = -2,     /* a CUDA runtime/driver call failed                    */
  CSK_ERR_DEVICE = -3,   /* a device-side check failed (bad expert id, bounded
                            wait ran out); the handle stays usable              */
  CSK_ERR_NOMEM = -4,    /* allocation failed or capacity exceeded               */
  CSK_ERR_MISSING = -5   /* an expert needed by the call was never loaded        */
} csk_status;

/* expert_mlp_node::activation_type (include/coalsack/nn/nn_ops/expert_mlp_node.h:27-30) */
enum { CSK_ACT_MODIFIED_SWIGLU = 0, CSK_ACT_STANDARD_SWIGLU = 1 };

/* Which expert kernel serves a forward call. AUTO picks by the number of
 * (token, expert) rows; the other two force one kernel (tests, benchmarks). */
enum {
  CSK_PATH_AUTO = 0,
  CSK_PATH_STREAM = 1,      /* weight-streaming kernel (few rows per expert)                    */
  CSK_PATH_TILE = 2,        /* tensor-core kernel, one CTA per work item                        */
  CSK_PATH_TILE_PAIR = 3    /* tensor-core kernel on CTA pairs (cta_group::2); needs cluster launch */
};

/* Layer description: graph_builder::config num_experts / expert_top_k /
 * use_sigmoid_gating / weight_before_ffn (include/coalsack/llm/graph_builder.h:29-44)
 * plus the per-node settings (moe_router_node.h:27-34, expert_mlp_node.h:44-52,
 * expert_merge_node.h:17-24). */
/* How the experts' weight matrices arrive:
 *   CSK_WEIGHTS_MXFP4  17-byte MXFP4 blocks (csk_moe_load_expert_mxfp4); both expert kernels.
 *   CSK_WEIGHTS_F16    fp16 row-major matrices (csk_moe_load_expert_f16): the reference's fp16 expert
 *                      slices (expert_mlp_node.h:533-647) and, with num_experts = top_k = 1, its dense
 *                      shared-expert FFN (dense_ffn_node.h:28-219).  Tensor-core kernel only. */
enum { CSK_WEIGHTS_MXFP4 = 0, CSK_WEIGHTS_F16 = 1 };

typedef struct csk_moe_config {
  int32_t num_experts;        /* E, experts of the whole layer                    */
  int32_t top_k;              /* k                                                */
  int32_t hidden;             /* H, multiple of 32                                */
  int32_t ffn;                /* F, multiple of 32                                */
  int32_t activation;         /* CSK_ACT_*                                        */
  int32_t has_bias;           /* experts carry b_up/b_gate/b_down                 */
  int32_t sigmoid_gating;     /* routing weight = sigmoid(logit) instead of softmax */
  int32_t weight_before_ffn;  /* scale the expert INPUT by the routing weight     */
  int32_t device;             /* CUDA device ordinal                              */
  int32_t expert_begin;       /* first expert resident on this device ...         */
  int32_t expert_count;       /* ... and how many (0 = all E); expert parallelism */
  int32_t weight_format;      /* CSK_WEIGHTS_MXFP4 (0, default) or CSK_WEIGHTS_F16         */
  int64_t max_tokens;         /* largest T (and, under expert parallelism, the
                                 largest number of received rows / k) of a call   */
} csk_moe_config;

typedef struct csk_moe_layer csk_moe_layer;

/* ---- lifetime ---------------------------------------------------------- */
int csk_moe_create(const csk_moe_config* cfg, csk_moe_layer** out);
int csk_moe_destroy(csk_moe_layer* layer);
/* Text of the last error on this handle (or of the last failed create when
 * layer is NULL).  Valid until the next call on the handle. */
const char* csk_moe_last_error(const csk_moe_layer* layer);
/* 1 when a usable CUDA device with compute capability 10.x is present. */
int csk_moe_device_ok(int device);

/* ---- weights ------------------------------------------------------------ */
/* Router weights Wg [E,H] fp32 row-major and optional bias [E] (host).
 * Replaces inputs 1 and 2 of moe_router_node (moe_router_node.h:51-124). */
int csk_moe_set_router(csk_moe_layer* layer, const float* gate_w, const float* gate_bias_or_null);

/* One expert's three MXFP4 matrices exactly as dynamic_mx_tensor::data_ptr()
 * holds them (w_up [F,H], w_gate [F,H], w_down [H,F]) and its fp32 biases (NULL
 * when has_bias = 0), all host pointers.  The matrices are repacked once into
 * the device tile layout.  Replaces what moe_weight_fetch_node hands to each
 * expert_mlp_node per frame (moe_weight_fetch_node.h:187-206,
 * src/llm/moe_weight_provider.cpp:160-188). */
int csk_moe_load_expert_mxfp4(csk_moe_layer* layer, int32_t expert_id, const uint8_t* w_up,
                              const uint8_t* w_gate, const uint8_t* w_down, const float* b_up,
                              const float* b_gate, const float* b_down);
/* A run of experts from the model's expert tensors: w_up / w_gate / w_down point at expert
 * `first_expert`'s slice of an [E, rows, cols] MXFP4 tensor (slices of rows*cols/32*17 bytes
 * one after the other, as the GGUF file holds ffn_{up,gate,down}_exps.weight and as
 * moe_weight_provider::get cuts them, src/llm/moe_weight_provider.cpp:160-188); the biases
 * at its row of the [E, n] bias tensors (:110, 194-199).  Copies of one expert overlap the
 * repack of the previous one.  This is the load-time path that makes a layer device-resident
 * instead of streaming experts per step through the host cache (src/llm/llm_engine.cpp:283-288). */
int csk_moe_load_experts_mxfp4(csk_moe_layer* layer, int32_t first_expert, int32_t count, const uint8_t* w_up,
                               const uint8_t* w_gate, const uint8_t* w_down, const float* b_up,
                               const float* b_gate, const float* b_down);
/* Expert weights as fp16 row-major matrices (layers created with CSK_WEIGHTS_F16): w_up and w_gate
 * [F,H], w_down [H,F], as dynamic_tensor holds FLOAT16 weights (dense_ffn_node.h:24, uint16 bit
 * patterns); biases fp32 or NULL as in csk_moe_load_expert_mxfp4. */
int csk_moe_load_expert_f16(csk_moe_layer* layer, int32_t expert_id, const uint16_t* w_up, const uint16_t* w_gate,
                            const uint16_t* w_down, const float* b_up, const float* b_gate, const float* b_down);

/* The same from fp32 matrices (dense_ffn_node also takes FLOAT32 weights, dense_ffn_node.h:58-62, 121-149):
 * rounded to fp16 (nearest even) on the device, since the tensor-core kernel's operands are fp16; the result
 * then differs from the reference's fp32 arithmetic by that rounding (2^-11 relative per weight, inside the
 * stated tolerance).  CSK_ERR_INVALID when a finite weight lies beyond the fp16 range. */
int csk_moe_load_expert_f32(csk_moe_layer* layer, int32_t expert_id, const float* w_up, const float* w_gate,
                            const float* w_down, const float* b_up, const float* b_gate, const float* b_down);

/* Expert slices in the GGUF block formats the reference's weight provider turns into fp16 on the host at
 * fetch time (src/llm/moe_weight_provider.cpp:120-159: Q4_K and Q6_K through dequantize_block_q4_K /
 * dequantize_block_q6_K, include/coalsack/gguf/gguf_dequant.h:147-261, then fp32_to_fp16, :458-489; F16 as
 * it is).  Here the raw blocks are copied to the device and decoded there, bit for bit the fp16 values the
 * provider would hand to expert_mlp_node.  For layers created with CSK_WEIGHTS_F16; each matrix has its own
 * type (ggml_type values, include/coalsack/gguf/gguf_types.h:24-39); a slice is hidden * ffn values, i.e.
 * hidden*ffn/256 super-blocks of 144 (Q4_K) or 210 (Q6_K) bytes.
 * f16_rounding: the reference's fp32_to_fp16 has two builds.  CSK_F16_TRUNCATE is the portable one its
 * CMake flags produce (mantissa truncated, NaN -> infinity, |x| < 2^-25 -> 0); CSK_F16_NEAREST is the F16C
 * one (round to nearest even; NaN payloads are not reproduced). */
enum { CSK_GGML_F16 = 1, CSK_GGML_Q4_K = 12, CSK_GGML_Q6_K = 14 };
enum { CSK_F16_TRUNCATE = 0, CSK_F16_NEAREST = 1 };
int csk_moe_load_expert_ggml(csk_moe_layer* layer, int32_t expert_id, int32_t type_up, const void* w_up,
                             int32_t type_gate, const void* w_gate, int32_t type_down, const void* w_down,
                             const float* b_up, const float* b_gate, const float* b_down, int32_t f16_rounding);
/* The decoders alone, host to host through the device: n_elements (a multiple of 256) values of Q4_K or
 * Q6_K blocks to fp16 bit patterns.  Errors go to csk_moe_last_error(NULL). */
int csk_moe_dequant_ggml_f16(int32_t device, int32_t ggml_type, const void* blocks, int64_t n_elements,
                         uint16_t* out_f16, int32_t f16_rounding);

/* The dense gated FFN of dense_ffn_node (dense_ffn_node.h:28-219: every token through the one weight
 * set, standard SwiGLU, biases optional) on a layer created with num_experts = top_k = 1,
 * CSK_WEIGHTS_F16 and CSK_ACT_STANDARD_SWIGLU: no router is involved.  hidden and out [T,H] fp32. */
int csk_moe_dense_forward(csk_moe_layer* layer, const float* hidden, int64_t T, float* out);
int csk_moe_dense_forward_dev(csk_moe_layer* layer, const float* d_hidden, int64_t T, float* d_out, void* stream);

/* The repacked weights of the resident experts as a file, and back: a later start of the same
 * layer (same shape, expert range and library build) skips the repack.  No counterpart in the
 * reference. */
int csk_moe_save_image(csk_moe_layer* layer, const char* path);
int csk_moe_load_image(csk_moe_layer* layer, const char* path);

/* Inverse of the repack: writes matrix `which` (0 up, 1 gate, 2 down from the
 * streaming kernel's layout; 3 up, 4 gate, 5 down from the tensor-core
 * kernel's layout) of a resident expert back as 17-byte blocks (host).  The
 * repack is lossless iff this returns the loaded bytes; the one rewrite is that
 * the streaming layout (which 0..2) stores scale byte 255 as 254, the value the
 * kernels read it as. */
int csk_moe_unpack_expert_mxfp4(csk_moe_layer* layer, int32_t expert_id, int32_t which,
                                uint8_t* out_blocks);
/* 1 if the expert's weights are resident on the device, 0 if not. */
int csk_moe_expert_resident(const csk_moe_layer* layer, int32_t expert_id);

/* ---- host-buffer entry points (what the reference nodes bind) ---------- */
/* moe_router_node::compute (moe_router_node.h:51-124, 140-214):
 * hidden [T,H] -> router_out [T,k,2]. */
int csk_moe_route(csk_moe_layer* layer, const float* hidden, int64_t T, float* router_out);

/* The whole layer: router (when router_out_in is NULL) -> dispatch by expert
 * -> grouped MXFP4 gated MLP -> weighted combine in router order.  Equals
 * moe_router_node + moe_weight_fetch_node + E x expert_mlp_node +
 * expert_merge_node (src/llm/llm_engine.cpp:721-753).  router_out_out
 * (optional) receives the routing actually used.  out is [T,H].
 * Large batches run as two passes over token ranges on three streams, so that
 * one range's copies overlap the other's kernels (same results: tokens are
 * independent); that only helps when the host buffers are page-locked --
 * copies from or to pageable memory block the calling thread. */
int csk_moe_forward(csk_moe_layer* layer, const float* hidden, int64_t T,
                    const float* router_out_in, float* router_out_out, float* out);

/* One expert_mlp_node (expert_mlp_node.h:392-530): dense [T,H] output with
 * zero rows for tokens that did not select expert_id.  *selected is set to 0
 * and out is left untouched when no token selected it (the reference then
 * emits a {0}-shaped tensor, :441-443), else to 1. */
int csk_moe_expert_forward(csk_moe_layer* layer, int32_t expert_id, const float* hidden, int64_t T,
                           const float* router_out, float* out, int32_t* selected);

/* expert_merge_node::compute (expert_merge_node.h:30-134): expert_outs[e] is a
 * dense [T,H] host buffer or NULL for an empty ({0}-shaped) input. */
int csk_moe_merge(csk_moe_layer* layer, const float* router_out, int64_t T,
                  const float* const* expert_outs, float* out);

/* ---- device-buffer entry points (no host copies; `stream` is a
 *      cudaStream_t passed as void*, NULL = the handle's own stream) ------- */
int csk_moe_route_dev(csk_moe_layer* layer, const float* d_hidden, int64_t T, float* d_router_out,
                      void* stream);
int csk_moe_forward_dev(csk_moe_layer* layer, const float* d_hidden, int64_t T,
                        const float* d_router_out_in, float* d_router_out_out, float* d_out,
                        void* stream);
/* The device-buffer calls only enqueue work.  csk_moe_sync waits for the last
 * one on this handle and reports what its kernels found (an expert id out of
 * range, rows routed to an expert that is not loaded, capacity exceeded). */
int csk_moe_sync(csk_moe_layer* layer);

/* ---- the layer with the steps either side of it ----------------------------
 * The reference runs an RMSNorm in front of the router and adds the layer's input
 * back after the merge (rmsnorm_node.h:20-83, eps 1e-5; src/llm/llm_engine.cpp:714-719
 * and 773-777); both are passes over [T,H] that cost a round trip each when they
 * are separate operators.  Here:  n = rmsnorm(x) * weight;  out = x + moe(n).
 * The norm reproduces the reference's sequential sum of squares, so the router sees
 * the reference's own input and its expert indices stay bit-exact; the residual is
 * one fp32 addition in the combine kernel.  set_ffn_norm takes a host weight [H]. */
int csk_moe_set_ffn_norm(csk_moe_layer* layer, const float* norm_weight, float eps);
int csk_moe_block_forward(csk_moe_layer* layer, const float* x, int64_t T, float* router_out_or_null, float* out);
int csk_moe_block_forward_dev(csk_moe_layer* layer, const float* d_x, int64_t T, float* d_router_out_or_null,
                              float* d_out, void* stream);
/* The same block with a shared expert (Llama-4 style, src/llm/llm_engine.cpp:755-777): out = x + (moe(n) + dense(n)),
 * n = rmsnorm(x) * weight, `shared` a layer as csk_moe_dense_forward takes (num_experts = top_k = 1, fp16 weight
 * format, same device and hidden size, weights loaded).  The dense FFN runs on the shared layer's own stream beside
 * the routed experts; the combine kernel adds its rows to the merge output, then the residual, in the reference's
 * order.  shared = NULL is csk_moe_block_forward. */
int csk_moe_block_forward_shared(csk_moe_layer* layer, csk_moe_layer* shared, const float* x, int64_t T,
                                 float* router_out_or_null, float* out);
int csk_moe_block_forward_shared_dev(csk_moe_layer* layer, csk_moe_layer* shared, const float* d_x, int64_t T,
                                     float* d_router_out_or_null, float* d_out, void* stream);

/* Routing for callers that must not allocate.  No counterpart in the reference
 * (its router keeps its logits in a std::vector on the host).
 *
 * Same result as csk_moe_route_dev, but it needs no handle and calls no
 * cudaMalloc/cudaFree or any other allocating routine: the [T,E] logits between
 * its two kernels live in a 1 MiB array compiled into this library's device
 * image.  Meant for hosts where device memory was handed out up front to one
 * owner (a serving process that reserves the whole GPU for its own pool, so a
 * later cudaMalloc simply fails) and for threads that may not block on the
 * allocator's device-wide synchronisation, such as a per-layer scheduler
 * thread that shares the GPU with other layers' streams.
 *
 * All pointers are device pointers on the CURRENT device: hidden [T,H] fp32,
 * gate_w [E,H] fp32, gate_bias [E] or NULL, router_out [T,k,2].  `stream` is a
 * cudaStream_t passed as void* (NULL = the default stream); the call only
 * enqueues work.
 * Limits: T*E <= 262144 logits (e.g. 2048 tokens at 128 experts), H a multiple
 * of 32, E <= 1024, k <= 16; beyond them the call returns CSK_ERR_NOMEM /
 * CSK_ERR_INVALID with a message in csk_moe_last_error(NULL) and launches nothing.
 * The first call on each device resolves the array's device address
 * (cudaGetSymbolAddress); make that first call before any stream capture.
 * The array is shared by every call in the process and keeps the last call's
 * logits; each call overwrites the part it reads, so nothing needs clearing,
 * but two calls that overlap on the same GPU (different streams or threads)
 * race on it: serialise them.
 * Every wait inside its kernels is bounded; one that runs out leaves that call's
 * router_out invalid and sets a status word that csk_moe_route_static_status
 * reports. */
int csk_moe_route_static(const float* d_hidden, int64_t T, int32_t H, const float* d_gate_w,
                         const float* d_gate_bias_or_null, int32_t E, int32_t k,
                         int32_t sigmoid_gating, float* d_router_out, void* stream);
/* CSK_OK, or CSK_ERR_DEVICE when a bounded wait ran out in a csk_moe_route_static
 * call on the current device since the last query (the word is cleared).  Call it
 * after synchronising the stream those calls ran on; it allocates nothing (one
 * 4-byte device-to-host copy).  No counterpart in the reference. */
int csk_moe_route_static_status(void);

/* ---- expert parallelism: the layer cut at its two exchange points -------
 * Rank r holds experts [expert_begin, expert_begin+expert_count).  A step is
 *   dispatch_dev  : route local tokens, group their (token, expert) rows by
 *                   global expert id (which is by destination rank, then
 *                   expert), write them as fp16 rows into d_send and the
 *                   per-expert row counts into d_counts [E] (int32)
 *   <all-to-all of counts, then of rows: the caller's NCCL>
 *   experts_dev   : run the resident experts over received rows.  d_recv holds
 *                   n_src segments (one per source rank), each ordered by local
 *                   expert; d_recv_counts is [n_src, expert_count] int32.
 *                   Output rows (fp32, [rows, H]) are written to d_ret in the
 *                   same order as d_recv.
 *   <all-to-all of output rows back>
 *   combine_dev   : weighted sum over k in router order of the returned rows
 *                   (d_back is in the order of d_send).
 * The reference has no counterpart (it runs every expert serially on one host
 * thread); the arithmetic per row is that of csk_moe_forward. */
/* Row pitch, in fp16 elements, of d_send / d_recv (H rounded up to 64). */
int csk_moe_ep_row_pitch(const csk_moe_layer* layer);
int csk_moe_ep_dispatch_dev(csk_moe_layer* layer, const float* d_hidden, int64_t T,
                            const float* d_router_out_in, void* d_send_f16, int32_t* d_counts,
                            void* stream);
int csk_moe_ep_experts_dev(csk_moe_layer* layer, const void* d_recv_f16,
                           const int32_t* d_recv_counts, int32_t n_src, int64_t total_rows,
                           float* d_ret, void* stream);
int csk_moe_ep_combine_dev(csk_moe_layer* layer, const float* d_back, int64_t T, float* d_out,
                           float* d_router_out_out, void* stream);
/* Expert placement for the csk_moe_ep_* stages.  Without a map the layer's
 * num_experts are both the router's experts and the slots that rows are grouped
 * by.  With a map the router has n_logical <= num_experts experts (set_router
 * then takes [n_logical, H] weights, router outputs carry logical ids) and
 * csk_moe_ep_dispatch_dev groups the rows of logical expert e under slot
 * primary_slot[e] -- or, for odd-numbered tokens, under replica_slot[e] when
 * that is >= 0 (a second copy of a heavily loaded expert on another rank).
 * Both arrays are [n_logical] int32 on the host; replica_slot may be null.
 * Slots must be distinct and below num_experts.  Call it before
 * csk_moe_set_router.  While a map is set, csk_moe_forward* (which group by the
 * router's own ids) are refused.  n_logical = 0 removes the map.
 * No counterpart in the reference. */
int csk_moe_ep_set_slot_map(csk_moe_layer* layer, int32_t n_logical, const int32_t* primary_slot,
                            const int32_t* replica_slot);

/* ---- expert parallelism over peer memory (NVLink) --------------------------
 * The same step without all-to-all collectives for the rows: dispatch writes each
 * row straight into the row buffer of the rank that owns its expert slot, at its
 * final expert-grouped position; the down projection's epilogue writes each output
 * row straight into the return buffer of the rank that owns the token.  What is
 * left for the caller's communication library is an all-gather of the per-slot
 * row counts and two barriers:
 *
 *   counts_dev   : route, map to slots, count this rank's rows per slot -> d_counts [E]
 *   <all-gather of d_counts into d_all_counts [world, E]>
 *   scatter_dev  : fp16 rows -> the owners' buffers (peer stores)
 *   <barrier>
 *   experts_dev  : resident experts over the received rows; fp32 output rows ->
 *                  the token owners' buffers (peer stores)
 *   <barrier>
 *   combine_dev  : weighted sum over k of the rows returned to this rank
 *
 * Setup, once: every rank exports three buffers as CUDA IPC handles (export),
 * the 3 * CSK_IPC_HANDLE_BYTES bytes of all ranks are gathered in rank order and
 * imported (import).  Ranks that live in one process exchange raw pointers
 * instead (local_ptrs / import_ptrs).  Rank r must own expert slots
 * [r*E/world, (r+1)*E/world) and all ranks must use the same max_tokens.
 * rows_hint: expected number of received rows (chooses the kernel; T*top_k when
 * the load is even).  No counterpart in the reference. */
#define CSK_IPC_HANDLE_BYTES 72 /* a CUDA IPC memory handle and the buffer's offset in that allocation */
int csk_moe_ep_p2p_export(csk_moe_layer* layer, uint8_t* handles /* 3 * CSK_IPC_HANDLE_BYTES */);
int csk_moe_ep_p2p_import(csk_moe_layer* layer, int32_t rank, int32_t world,
                          const uint8_t* all_handles /* world * 3 * CSK_IPC_HANDLE_BYTES */);
int csk_moe_ep_p2p_local_ptrs(csk_moe_layer* layer, void** x16, void** info, void** back);
int csk_moe_ep_p2p_import_ptrs(csk_moe_layer* layer, int32_t rank, int32_t world, void* const* x16,
                               void* const* info, void* const* back);
/* The gather of the counts and the two barriers without a collective library: flags in a sync
 * area every peer can write (it rides at the tail of the return buffer, so the handles above
 * cover it).  which = 0 with d_counts [E] -> d_all_counts [world, E] replaces the all-gather;
 * which = 1 / 2 with null pointers are the two barriers.  Every rank must call the same sequence.
 * The wait inside is bounded (a few seconds); when it runs out csk_moe_sync reports
 * CSK_ERR_DEVICE.  Only for ranks on DIFFERENT GPUs: ranks emulated on one GPU must not wait on
 * one another's kernels (run their stages in lockstep instead). */
int csk_moe_ep_p2p_sync_dev(csk_moe_layer* layer, int32_t which, const int32_t* d_counts, int32_t* d_all_counts,
                            void* stream);
int csk_moe_ep_p2p_counts_dev(csk_moe_layer* layer, const float* d_hidden, int64_t T,
                              const float* d_router_out_in, int32_t* d_counts, void* stream);
int csk_moe_ep_p2p_scatter_dev(csk_moe_layer* layer, const float* d_hidden, int64_t T,
                               const int32_t* d_all_counts, void* stream);
int csk_moe_ep_p2p_experts_dev(csk_moe_layer* layer, const int32_t* d_all_counts, int64_t rows_hint,
                               void* stream);
int csk_moe_ep_p2p_combine_dev(csk_moe_layer* layer, int64_t T, float* d_out, float* d_router_out_out,
                               void* stream);

/* ---- knobs and observability ------------------------------------------- */
int csk_moe_set_path(csk_moe_layer* layer, int32_t path /* CSK_PATH_* */);

/* The gated activation and where the routing weight is applied -- the per-node settings
 * expert_mlp_node::set_activation_type / set_weight_before_ffn (expert_mlp_node.h:44-52) --
 * changed on an existing handle (the weights stay resident). */
int csk_moe_set_activation(csk_moe_layer* layer, int32_t activation /* CSK_ACT_* */, int32_t weight_before_ffn);

/* How the router reaches the reference's selection (moe_router_node.h:161-177: each
 * logit a sequential fp32 multiply-then-add chain over the hidden dimension, top-k by
 * logit).  Every mode returns the same expert indices as the reference, bit for bit.
 *   CSK_ROUTER_CHAIN: every logit by the reference's own chain (one launch).
 *   CSK_ROUTER_CERTIFIED: logits by fused multiply-adds in 32-column blocks with a
 *     rigorous bound on their distance from the chain's value; a token whose k+1 best
 *     logits are further apart than the bounds keeps that selection, any other token is
 *     recomputed by the chain.  Routing WEIGHTS of certified tokens come from the fast
 *     logits and differ from the reference's by a few ulp (below 1e-6).
 *   CSK_ROUTER_AUTO (default): certified for batches of up to 4 tokens, where the chain
 *     is one long dependency on a few SMs; the chain kernel for anything larger, where it
 *     is the faster of the two (measured). */
enum { CSK_ROUTER_AUTO = 0, CSK_ROUTER_CHAIN = 1, CSK_ROUTER_CERTIFIED = 2 };
int csk_moe_set_router_mode(csk_moe_layer* layer, int32_t mode);
/* Tokens routed in certified mode since the handle was created, and how many of them
 * had to be recomputed by the chain (waits for the device). */
int csk_moe_get_router_stats(csk_moe_layer* layer, int64_t* routed_tokens, int64_t* chain_tokens);

/* Device time of the stages of the last forward call on this handle, in
 * milliseconds (CUDA events on the stream the kernels ran on).  Collection is
 * off by default; csk_moe_enable_timing(layer, 1) turns it on. */
typedef struct csk_moe_timings {
  float route_ms;    /* router kernel                                  */
  float permute_ms;  /* histogram, scan, scatter + fp16 gather         */
  float gate_up_ms;  /* first grouped contraction + activation         */
  float down_ms;     /* second grouped contraction                     */
  float combine_ms;  /* weighted sum over k                            */
  float total_ms;    /* first to last kernel                           */
  int32_t path;      /* CSK_PATH_STREAM or CSK_PATH_TILE actually used */
  int32_t launches;  /* kernels launched by the call                   */
} csk_moe_timings;
int csk_moe_enable_timing(csk_moe_layer* layer, int32_t on);
int csk_moe_get_timings(csk_moe_layer* layer, csk_moe_timings* out);

/* Counters of the last forward call: rows routed to each expert (E int64,
 * host), number of distinct experts hit, weight bytes those experts hold. */
int csk_moe_get_counters(csk_moe_layer* layer, int64_t* rows_per_expert, int64_t* distinct_experts,
                         int64_t* weight_bytes_streamed);

/* ---- test hooks ------------------------------------------------------------
 * For the tests of the failure path (the reference reports failures as values,
 * expert_mlp_node.h:139-146; here a kernel that gives up reports through the
 * status word and the handle stays usable).  Nothing here faults or hangs the GPU.
 *   CSK_DEBUG_WAIT_BUDGET         clock cycles a device-side wait may take before it
 *                                 gives up (default 2e9, about a second); applies to
 *                                 every handle on the device
 *   CSK_DEBUG_STALL_TILE_PRODUCER non-zero: in the NEXT tensor-core expert launch the
 *                                 copy role issues nothing, so every other role's wait
 *                                 runs out, the kernel tears down and the call reports
 *                                 CSK_ERR_DEVICE (one shot) */
enum { CSK_DEBUG_WAIT_BUDGET = 0, CSK_DEBUG_STALL_TILE_PRODUCER = 1 };
int csk_moe_debug_set(csk_moe_layer* layer, int32_t key, int64_t value);

#ifdef __cplusplus
}
#endif
#endif /* CSK_MOE_H */
