/*
 * glmflash_b200 -- C ABI of the B200 (sm_100a) EXL3 MoE expert path.
 *
 * The library is a drop-in for the routed-expert hot path of cuylerstuwe/glm-flash-rs.  Upstream, Rust
 * owners (`ExpertGpu`, `FastExperts`, `Grouping`, `Moe`) allocate scratch through the CUDA driver and
 * launch precompiled kernels by symbol (src/cuda.rs:657-757).  Here each owner is an opaque handle
 * behind plain-C entry points; a Rust (or any other) host binds them with `extern "C"` exactly as
 * upstream binds its other native libraries (native/roce_bridge.cpp:22-104, src/roce.rs:89-141).
 *
 * Conventions (the same as upstream's native bridges):
 *   - every call returns 0 on success and -1 on failure; the message of the last failure on the calling
 *     thread is glmflash_error();  no exception, trap or exit crosses the boundary;
 *   - handles are single-owner: no concurrent calls on one handle;
 *   - run functions only enqueue work on the caller's stream: they never synchronise, allocate or read
 *     back, and may be captured into a CUDA graph and replayed (src/experts.rs:309-316,
 *     src/fast_experts.rs:383-412);
 *   - the handle owns scratch and outputs (zero-initialised at construction, src/experts.rs:395-429); the
 *     caller owns weights, inputs, routing tables and the stream; outputs stay valid until the next run on
 *     the handle;
 *   - all pointers are device pointers unless a name ends in `_host`;
 *   - there is no CPU fallback: without a CUDA device every constructor fails.
 *
 * Tensor layouts (src/experts.rs:146-156 with the model sizes as parameters):
 *   gt, ut  uint32 [E1][H/16][I/16][32]   trellis tiles of the gate / up projections (H -> I)
 *   dt      uint32 [E1][I/16][H/16][32]   trellis tiles of the down projection (I -> H)
 *   suh_g, suh_u fp16 [E1][H];  suh_d fp16 [E1][I]     input sign/scale vectors
 *   svh_g, svh_u fp16 [E1][I];  svh_d fp16 [E1][H]     output sign/scale vectors
 * E1 = experts + 1: the shared expert is expert id `experts` (the last bank entry).
 *   picks   int32 [rows][slots]: slots-1 distinct routed ids, then the shared id `experts`
 *   ids     int32 [E1], count int32 [1], members int32 [E1][maxm]   (the grouping, native/grouping.cu)
 *           member code = row * 32 + slot, ascending rows first, -1 padded
 *   pair index p = row * slots + slot  (native/exl3.cu:160-166,228-231)
 */
#ifndef GLMFLASH_B200_H
#define GLMFLASH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GLMFLASH_ABI_VERSION 1

/* Model sizes and policy of one expert bank.  Passed by pointer with its size (glmflash_config_bytes)
 * so that host and library can detect a layout mismatch (native/roce_bridge.cpp:29, src/roce.rs:137-141). */
typedef struct glmflash_config {
    int32_t hidden;        /* H: model width, multiple of 256 (upstream 4096; benchmark 2048)             */
    int32_t inter;         /* I: expert intermediate width, multiple of 256 (upstream 512/rank; 1536)      */
    int32_t experts;       /* E: routed experts; the shared expert has id E                                */
    int32_t slots;         /* S: top-k + 1 (upstream 9; benchmark 5), at most 32                            */
    int32_t max_rows;      /* scratch capacity in rows                                                     */
    int32_t shared_exl3;   /* 1: the shared expert (id E) is an EXL3 expert of the bank and is computed here;
                              0: upstream behaviour, ids >= E are skipped (native/exl3.cu:151);
                              2: expert parallel, handles of <= 16 rows: decided per window on the device -- of the
                                 ranks (equal contiguous expert windows, rank = expert_lo / window size) the one whose
                                 window holds the fewest distinct routed experts of the routing table computes it
                                 (ties: the lowest rank); every rank evaluates the same table, so all agree       */
    int32_t expert_lo;     /* expert-parallel window: of the routed experts only ids in [expert_lo,        */
    int32_t expert_hi;     /* expert_hi) are computed here (0, E = all of them)                            */
    float   limit;         /* SwiGLU clamp (upstream 10.0, src/experts.rs:521)                             */
    int32_t pdl;           /* 1: chain the kernels of a run with programmatic dependent launch, so that each
                              kernel's weight prefetch overlaps its predecessor's tail (upstream's "pdl" load
                              policy, src/experts.rs:350-354, native/expert_loads.cu:38-44); 0: plain launches */
    int32_t shared_row_lo; /* expert-parallel prefill: with shared_exl3 = 1 the shared expert is computed here only   */
    int32_t shared_row_hi; /* for window rows in [shared_row_lo, shared_row_hi) (0, 0 = every row); handles for more
                              than 16 rows only                                                              */
    int32_t reserved[4];
} glmflash_config;

/* The nine tensors `m.pointer(..moe.experts.*)` resolves upstream (src/experts.rs:467). */
typedef struct glmflash_weights {
    const uint32_t *gt, *ut, *dt;
    const uint16_t *suh_g, *suh_u, *suh_d;
    const uint16_t *svh_g, *svh_u, *svh_d;
} glmflash_weights;

int         glmflash_abi_version(void);
size_t      glmflash_config_bytes(void);
size_t      glmflash_weights_bytes(void);
const char *glmflash_error(void);                 /* last error of this thread ("" if none) */

/* ---- trellis decode and a single EXL3 linear (building blocks; parity probes) --------------------- */

/* Decode `tiles` 16x16 tiles: words [tiles][32] -> out fp16 [tiles][16][16] (row k, column n), bit-exact
 * with upstream's decode (native/exl3.cu:21-40 <=> src/experts.rs:43-74). */
int glmflash_exl3_decode(void *stream, const uint32_t *words, int64_t tiles, uint16_t *out);

/* y[rows][N] fp16 = H(fp16(H(x*suh)/sqrt128) @ W_q)/sqrt128 * svh for fp16 x[rows][K], rows <= 16
 * (one matrix of src/experts.rs:100-135).  scratch: at least glmflash_exl3_linear_scratch_bytes(K,N). */
size_t glmflash_exl3_linear_scratch_bytes(int K, int N);
int glmflash_exl3_linear(void *stream, const uint16_t *x, int rows, const uint32_t *words, const uint16_t *suh,
                         const uint16_t *svh, int K, int N, uint16_t *y, void *scratch);

/* The same linear for callers that cannot allocate device memory.  This entry point has no counterpart in the
 * reference.  It exists for hosts that took over the whole device heap at start-up (so a later cudaMalloc by a
 * library would fail or fragment their pool) and for serving loops where an allocator call would stall every
 * stream of the device.  The scratch is a fixed array inside the library (glmflash_exl3_linear_static_max_bytes(),
 * 132 KiB, held by every GPU that loads the library until the process exits), so shapes are limited to
 * K <= 4096; larger shapes are rejected with an error.  The call itself allocates nothing.
 * The first call on a device looks up the array's device address (a one-time, per-device set-up step): make that
 * first call outside any stream capture.  All calls share the one array and it keeps the previous call's
 * contents; the call clears what has to start at zero, but two calls that overlap on the GPU (different streams
 * without ordering, or different host threads) race on it: order them. */
size_t glmflash_exl3_linear_static_max_bytes(void);
int glmflash_exl3_linear_static(void *stream, const uint16_t *x, int rows, const uint32_t *words, const uint16_t *suh,
                                const uint16_t *svh, int K, int N, uint16_t *y);

/* ---- Grouping  (src/grouping.rs:29-111; kernels native/grouping.cu) --------------------------------- */
typedef struct glmflash_grouping glmflash_grouping;
int  glmflash_grouping_new(const glmflash_config *cfg, size_t cfg_bytes, glmflash_grouping **out);
void glmflash_grouping_free(glmflash_grouping *g);
/* Grouping::run(s, picks, rows): fills ids / count / members ([E1][max_rows]).  1 <= rows <= max_rows. */
int  glmflash_grouping_run(glmflash_grouping *g, void *stream, const int32_t *picks, int rows);
const int32_t *glmflash_grouping_ids(const glmflash_grouping *g);
const int32_t *glmflash_grouping_count(const glmflash_grouping *g);
const int32_t *glmflash_grouping_members(const glmflash_grouping *g);

/* ---- ExpertGpu: decode / verify windows of 1..16 rows  (src/experts.rs:365-563) --------------------- */
typedef struct glmflash_experts glmflash_experts;
/* ExpertGpu::new_rows(d, native, max_rows); max_rows in 1..16 (src/experts.rs:391-394). */
int  glmflash_experts_new(const glmflash_config *cfg, size_t cfg_bytes, glmflash_experts **out);
void glmflash_experts_free(glmflash_experts *e);
/* ExpertGpu::run_rows(stream, .., input, picks, ids, count, members, rows, maxm).  input: bf16
 * [rows][x_stride].  Bounds as upstream: 1 <= rows <= max_rows, rows <= maxm <= max_rows
 * (src/experts.rs:461-464).  Result: glmflash_experts_y() = Y fp32 [rows*slots][H]; rows of pairs whose
 * expert is skipped (shared_exl3 = 0, or outside the expert window) are left untouched. */
int  glmflash_experts_run_rows(glmflash_experts *e, void *stream, const glmflash_weights *w, const void *input,
                               int x_stride, const int32_t *picks, const int32_t *ids, const int32_t *count,
                               const int32_t *members, int rows, int maxm);
float *glmflash_experts_y(const glmflash_experts *e);
/* Down-projection inputs Xd fp16 [rows*slots][I] of the last run (upstream's `xd`; probes compare it). */
const uint16_t *glmflash_experts_xd(const glmflash_experts *e);
/* Device status word (int32): 0 after a clean run; non-zero when a bounded wait inside a kernel gave up
 * (the analogue of upstream's poison word, native/roce.cu:127-141).  Read it after synchronising. */
const int32_t *glmflash_experts_status(const glmflash_experts *e);
/* Clears the status word (and the arrival counters a give-up may have left half way), in stream order: the way back
 * to a usable owner after a bounded wait ran out (upstream rebuilds its transport after a poisoned exchange,
 * src/roce.rs:275-282). */
int  glmflash_experts_clear_status(glmflash_experts *e, void *stream);
/* Profiling aid in the spirit of upstream's PROBE modes (native/expert_loads.cu:46-47): run only the selected
 * kernels of the pipeline (1 = input rotation, 2 = gate/up GEMV + SwiGLU epilogue, 4 = down GEMV + epilogue;
 * default 7).  Skipped phases leave the scratch of the previous run in place; results are then meaningless. */
int  glmflash_experts_set_phases(glmflash_experts *e, int mask);

/* ---- FastExperts: prefill chunks of up to 8192 rows  (src/fast_experts.rs:27-208) ------------------- */
typedef struct glmflash_fast_experts glmflash_fast_experts;
int  glmflash_fast_experts_new(const glmflash_config *cfg, size_t cfg_bytes, glmflash_fast_experts **out);
void glmflash_fast_experts_free(glmflash_fast_experts *f);
/* FastExperts::run(s, .., input, picks, ids, count, members, rows, maxm, shared_x).  shared_x != 0 when
 * suh_g == suh_u so one rotated copy of the input serves both projections (src/batch.rs:195-201). */
int  glmflash_fast_experts_run(glmflash_fast_experts *f, void *stream, const glmflash_weights *w,
                               const void *input, int x_stride, const int32_t *picks, const int32_t *ids,
                               const int32_t *count, const int32_t *members, int rows, int maxm, int shared_x);
float *glmflash_fast_experts_output(const glmflash_fast_experts *f);       /* fp32 [rows*slots][H], pair order */
/* Down-projection inputs of the last run, fp16 [grouped rows][I].  The prefill path keeps its intermediate rows
 * GROUPED (the rows of an expert are contiguous, experts in ascending id order, so that an M tile is one TMA
 * tensor load); grouped row j belongs to pair glmflash_fast_experts_row_pairs()[j]; the number of grouped rows
 * is plan[1], the number of 128-row M tiles plan[0]. */
const uint16_t *glmflash_fast_experts_xd(const glmflash_fast_experts *f);
const int32_t *glmflash_fast_experts_row_pairs(const glmflash_fast_experts *f);
const int32_t *glmflash_fast_experts_plan(const glmflash_fast_experts *f);
/* Device status word, as glmflash_experts_status. */
const int32_t *glmflash_fast_experts_status(const glmflash_fast_experts *f);
int  glmflash_fast_experts_clear_status(glmflash_fast_experts *f, void *stream);
/* Profiling aid, as glmflash_experts_set_phases: 1 = plan, 2 = input rotation, 4 = gate/up GEMM, 8 = down GEMM
 * (default 15). */
int  glmflash_fast_experts_set_phases(glmflash_fast_experts *f, int mask);

/* ---- Moe: the whole layer after routing  (src/moe.rs:11-182, src/batch.rs:1160-1210) ---------------- */
typedef struct glmflash_moe glmflash_moe;
/* max_rows <= 16 builds the decode / verify pipeline, larger the prefill pipeline.
 * Windows of <= 16 rows run as three launches per layer (gate/up with grouping and input rotation inside, down,
 * combine: upstream's router-to-combine sequence src/moe.rs:101-181 in three kernels instead of eight).  With the
 * environment variable GLMFLASH_LAYER_KERNELS=1 (read at construction) they run as ONE kernel per layer, which also
 * carries the cross-GPU exchange of glmflash_moe_run_ep; on one GPU it measured slower than the three launches. */
int  glmflash_moe_new(const glmflash_config *cfg, size_t cfg_bytes, glmflash_moe **out);
void glmflash_moe_free(glmflash_moe *m);
/* group -> routed and shared experts -> combine:
 *   out[r][:] = sum_{s < slots-1} route_w[r][s] * Y[r][s][:] + Y[r][slots-1][:]     (fp32 [rows][H])
 * With an expert window the sum covers this GPU's experts only (a partial for the cross-GPU sum).
 * route_w: fp32 [rows][slots] (the last entry of a row is not read). */
int  glmflash_moe_run(glmflash_moe *m, void *stream, const glmflash_weights *w, const void *input, int x_stride,
                      const int32_t *picks, const float *route_w, int rows);
float *glmflash_moe_output(const glmflash_moe *m);
/* The pair results Y fp32 [rows*slots][H] behind the last run (the ExpertGpu / FastExperts output of this owner). */
const float *glmflash_moe_pairs(const glmflash_moe *m);
/* Device status word of the owner behind this layer (glmflash_experts_status / glmflash_fast_experts_status), and its
 * reset. */
const int32_t *glmflash_moe_status(const glmflash_moe *m);
int  glmflash_moe_clear_status(glmflash_moe *m, void *stream);
/* Profiling aid: 1 = grouping, 2 / 4 / 8 = the three ExpertGpu phases above, 16 = combine (default 31).  For
 * windows of <= 16 rows grouping and input rotation are fused into the gate/up kernel (bits 1 and 2 select nothing). */
int  glmflash_moe_set_phases(glmflash_moe *m, int mask);
/* Host-buffer convenience used by the end-to-end measurement: copies input / picks / route_w from host
 * memory, runs, copies out[rows][H] back, and synchronises the stream. */
int  glmflash_moe_run_host(glmflash_moe *m, void *stream, const glmflash_weights *w, const void *input_host,
                           int x_stride, const int32_t *picks_host, const float *route_w_host, int rows,
                           float *out_host);

/* PDL contract (config.pdl = 1): how a host kernel joins the chain at either edge of a layer, as upstream chains its own
 * kernels around the expert loads (native/expert_loads.cu:38-44, src/experts.rs:350-354).  The kernels of a window of
 * <= 16 rows, and the grouping, router, combine and exchange kernels of every window, are launched with the
 * programmatic-stream-serialization attribute and execute griddepcontrol.wait in every CTA that does work, so "the
 * kernel before has completed" is transitive along the stream; the plan / rotation / GEMM kernels in the middle of a
 * prefill layer are plain launches (fully ordered).
 *   In front of a layer (the producer of `input`, `picks`, `route_w`): nothing is required.  The first kernel of
 *     glmflash_moe_run / glmflash_moe_run_ep / glmflash_route touches no global memory before its griddepcontrol.wait, so
 *     the producer may be a plain kernel, or call griddepcontrol.launch_dependents as early as it likes (the layer's CTAs
 *     then become resident and set up their barriers while the producer drains).
 *   Behind a layer (a consumer of glmflash_moe_output / glmflash_ep_output), when the consumer is itself launched with the
 *     attribute: the layer's last kernel calls griddepcontrol.launch_dependents at its start, so the consumer's CTAs may
 *     start while the layer's last kernel (with GLMFLASH_LAYER_KERNELS=1: the whole layer) is still running.  Before its own
 *     griddepcontrol.wait the consumer may read its own weights and any buffer the layer does not write (a prefetch);
 *     it must not read the layer's output, pair buffer or status word, and must not write `input`, `picks`, `route_w`
 *     or the weights.  After the wait everything the layer wrote is visible.
 *   A consumer launched without the attribute is ordered after the whole layer, as any kernel in the stream. */

/* ---- expert-parallel combine over NVLink ------------------------------------------------------------ */
/* One owner per rank (one process per GPU).  It replaces upstream's gather + ordered sum after the MoE layer
 * (src/model.rs:485-496; Nccl::all_gather_f32 src/comm.rs:261-285 / Roce::gather src/roce.rs:283-330) by ONE kernel
 * per rank: combine this rank's pairs, store the partial into every peer's receive slot over NVLink (peer-mapped
 * memory, plain stores), signal, wait (bounded) for the peers' partials and add the slots in rank order.
 * Set-up mirrors upstream's bootstrap (src/comm.rs:109-162): every rank creates its owner, publishes an opaque
 * handle of glmflash_ep_handle_bytes() bytes, receives all ranks' handles (in rank order, by whatever channel the
 * host has: TCP, torch.distributed, ...) and calls glmflash_ep_connect once.  The handle carries a hash of the sizes the
 * peers' address arithmetic depends on (hidden, inter, experts, slots, max_rows, world): connect fails, before mapping
 * anything, when a rank was built differently (upstream's config agreement, src/comm.rs:66-96, src/model.rs:259-315).  Every rank must then call
 * glmflash_ep_combine the same number of times in the same order.  A peer that never arrives makes the wait give up
 * after a bounded number of polls: the status word becomes non-zero and the output of that call is undefined. */
typedef struct glmflash_ep glmflash_ep;
size_t glmflash_ep_handle_bytes(void);
int  glmflash_ep_new(const glmflash_config *cfg, size_t cfg_bytes, int rank, int world, glmflash_ep **out);
void glmflash_ep_free(glmflash_ep *h);
int  glmflash_ep_get_handle(glmflash_ep *h, void *handle_out);
int  glmflash_ep_connect(glmflash_ep *h, const void *all_handles /* world x handle_bytes, rank order */);
/* Y: fp32 [rows*slots][H] pair results of this rank (glmflash_moe_pairs); the config's expert window decides which
 * routed pairs are this rank's, shared_here whether the shared expert's pair is (it may move from layer to layer):
 * 1 / 0, or 2 = decided per window on the device by the rule of config.shared_exl3 = 2 (windows of <= 16 rows).
 * Result: glmflash_ep_output() fp32 [rows][H]. */
int  glmflash_ep_combine(glmflash_ep *h, void *stream, const float *Y, const int32_t *picks, const float *route_w, int rows,
                         int shared_here);
float *glmflash_ep_output(const glmflash_ep *h);
/* The layer and its exchange in one call (upstream: Moe::run_prefetched followed by finish(), src/model.rs:634-639).
 * With the one-launch layer kernel selected (GLMFLASH_LAYER_KERNELS=1) windows of <= 16 rows take ONE launch per rank:
 * the layer kernel stores each finished 128-column block of this rank's partial straight into every peer's receive slot
 * and adds the ranks' slots in rank order itself; otherwise, and for larger windows, the experts run and then
 * glmflash_ep_combine.  shared_here: 1 / 0 = this rank computes / skips the shared
 * expert in this call, 2 = decided per window on the device (the layer owner's config must say 2 as well), -1 = as the
 * layer owner's config says.  Result: glmflash_ep_output(). */
int  glmflash_moe_run_ep(glmflash_moe *m, glmflash_ep *ep, void *stream, const glmflash_weights *w, const void *input,
                         int x_stride, const int32_t *picks, const float *route_w, int rows, int shared_here);
const int32_t *glmflash_ep_status(const glmflash_ep *h);
/* A peer time-out leaves the status word set, and while it is set every later wait gives up at once (a dead peer costs
 * one time-out, not one per block).  Clear it, in stream order, once the host has dealt with the failure. */
int  glmflash_ep_clear_status(glmflash_ep *h, void *stream);
/* Windows of more than 16 rows: send the ranks' partial rows as bf16 instead of fp32 (upstream casts the rows to bf16
 * before its prefill gather and adds them in fp32, src/batch.rs:651-658).  Every rank must choose the same.  Default 0:
 * fp32, whose result has the bytes of an fp32 all-gather + rank-ordered sum.  With 1 every partial, the owner's own
 * included, is rounded to bf16 once before the fp32 sum in rank order; the finished rows stay fp32. */
int  glmflash_ep_set_exchange_bf16(glmflash_ep *h, int on);
/* Number of polls after which a wait for a peer gives up (default 2,000,000, about a second). */
int  glmflash_ep_set_wait_limit(glmflash_ep *h, uint32_t polls);
/* For a host that drives several GPUs from ONE process (peer access enabled by the host): connect with the peers'
 * glmflash_ep_local_base() pointers instead of IPC handles. */
void *glmflash_ep_local_base(const glmflash_ep *h);
int  glmflash_ep_connect_ptrs(glmflash_ep *h, void *const *peer_bases /* world entries, own entry ignored */);
/* out[r][:] = sum over ranks (ascending rank order) of gathered[rank][r][:], the fixed-order sum upstream
 * applies after its all-gather (src/model.rs:485-496, src/comm.rs:1-2).  gathered: fp32 [world][rows][H]. */
int glmflash_rank_sum(void *stream, const float *gathered, int world, int rows, int hidden, float *out);

/* ---- router next to the path (upstream call sites src/moe.rs:77-111, src/window_ops.rs:159-199) -------------------
 * Upstream runs precompiled kernels without published source here, so these two follow the benchmark's definition
 * of the router and their parity with upstream is not pinned.  Both only enqueue work (graph-capturable);
 * pdl != 0 chains them with programmatic dependent launch like the expert kernels.
 * logits[r][e] = sum_k x[r][k] * wr[e][k]: x bf16 [rows][x_stride >= hidden], wr bf16 [experts][hidden], logits fp32
 * [rows][experts], fp32 accumulation. */
int glmflash_router_logits(void *stream, const uint16_t *x, int x_stride, const uint16_t *wr, int rows, int hidden,
                           int experts, float *logits, int pdl);
/* Sigmoid top-k: per row the topk largest logits (ties to the lower expert id) in descending order,
 * weight = sigmoid(logit) / sum of the chosen sigmoids; the last slot names the shared expert (id = experts) with
 * weight 1.  picks int32 [rows][topk + 1], weights fp32 [rows][topk + 1]: the routing table glmflash_moe_run takes. */
int glmflash_topk(void *stream, const float *logits, int rows, int experts, int topk, int32_t *picks, float *weights,
                  int pdl);
/* Both steps: windows of <= 16 rows take ONE launch (a CTA per row computes the row's logits and selects), larger
 * windows the two kernels above.  logits (fp32 [rows][experts], caller's) receives the logits in both cases. */
int glmflash_route(void *stream, const uint16_t *x, int x_stride, const uint16_t *wr, int rows, int hidden, int experts,
                   int topk, float *logits, int32_t *picks, float *weights, int pdl);

/* ---- prepared weights  (src/prepared.rs:15-377; layout: docs/ARTIFACTS.md "Prepared target") ---------------------
 * A prepared model is a JSON manifest (format 1: file size, chunk size, one SHA-256 per chunk, storage table, object
 * tree with tensor leaves, preparation key) next to its payload `data.bin`.  open parses and validates the manifest
 * (Prepared::open_parts: chunk bound 128 MiB, hash count, payload size, ordered storages inside the payload, every
 * tensor inside its storage and on its storage's device); it needs no GPU.  Tensor paths are upstream's:
 * `weights.layers[3].moe.experts.gt` (fields '.', sequences '[i]', dict keys '[key]').  The model-specific checks of
 * Prepared::open (model name, rank / world, geometry) are the host's: glmflash_prepared_key_int reads the key. */
typedef struct glmflash_prepared glmflash_prepared;
typedef struct glmflash_tensor_info {
    char    dtype[16];     /* "int32", "float16", ... (src/prepared.rs:42-50)                                  */
    int32_t rank;          /* at most 8                                                                        */
    int32_t on_device;     /* 1: the tensor's storage is a CUDA storage                                        */
    int32_t contiguous;    /* 1: dense row-major strides (Prepared::expect)                                    */
    int32_t reserved;
    int64_t shape[8], stride[8];   /* elements                                                                 */
    int64_t nbytes;        /* from the first to the end of the last element                                    */
    void   *ptr;           /* after glmflash_prepared_load: device (or host, for cpu storages) address; else NULL */
} glmflash_tensor_info;
int  glmflash_prepared_open(const char *manifest_path, glmflash_prepared **out);
void glmflash_prepared_close(glmflash_prepared *p);
int  glmflash_prepared_key_int(const glmflash_prepared *p, const char *name, int64_t *value);
int  glmflash_prepared_tensor_count(const glmflash_prepared *p);
const char *glmflash_prepared_tensor_name(const glmflash_prepared *p, int i);          /* sorted paths */
int  glmflash_prepared_tensor(const glmflash_prepared *p, const char *name, glmflash_tensor_info *info);   /* Loaded::pointer */
/* Reads the whole payload and checks every chunk against its SHA-256 (no GPU). */
int  glmflash_prepared_verify(glmflash_prepared *p);
/* Prepared::load_selected: uploads the storages that hold a tensor whose path starts with one of the prefixes (all of
 * them when n_prefixes == 0); every chunk that is read is verified first.  Allocates and synchronises: a set-up call. */
int  glmflash_prepared_load(glmflash_prepared *p, const char *const *prefixes, int n_prefixes);

/* Upstream shards every expert four ways by tensor parallelism: a rank's `...moe.experts.{gt,ut}` hold 512 of the
 * intermediate's columns, `dt` the matching 512 rows, `suh_d / svh_g / svh_u` the matching slices (src/experts.rs:146-156).
 * This puts the slices of the experts [e_lo, e_hi) back together (device copies on `stream`), so that an expert-parallel
 * rank owns whole experts.  shards: the n_shards ranks' manifests in rank order, the tensors under `stem` loaded on the
 * current device.  glmflash_expert_bank_weights gives the nine pointers in the form the owners take (indexed by the
 * GLOBAL expert id: only ids of the window may be touched -- configure expert_lo / expert_hi accordingly, and
 * shared_exl3 = 0: upstream's shared expert is not an EXL3 expert) and the re-assembled sizes. */
typedef struct glmflash_expert_bank glmflash_expert_bank;
int  glmflash_expert_bank_from_tp(glmflash_prepared *const *shards, int n_shards, const char *stem, int e_lo, int e_hi, void *stream,
                                  glmflash_expert_bank **out);
int  glmflash_expert_bank_weights(const glmflash_expert_bank *b, glmflash_weights *w, int32_t *hidden, int32_t *inter);
void glmflash_expert_bank_free(glmflash_expert_bank *b);

/* ---- verify-window graph cache  (src/verifier_graph_cache.rs; used by src/multi_decode.rs:470-537) ----------------
 * Upstream captures one CUDA graph per (slot, parity, rows, geometry) of its speculative-verify windows -- two to four
 * requests share one <= 16-row expert call -- and keeps them under two caps.  The same policy: action() says replay,
 * run eagerly (a bounded cache captures a key only from its `after`-th sighting on) or capture; insert() retains a
 * captured graph, evicting least recently used entries while there are `entries` of them or more than `nodes` graph
 * nodes; a graph that alone exceeds `nodes` is handed back.  The unbounded policy clears everything when it is full.
 * key: any 64-bit value the host derives from the window's shape, e.g. rows | parity << 8 | slot << 16. */
typedef struct glmflash_graph_policy {
    int32_t  bounded;      /* 1: upstream's ALASKA_VERIFY_GRAPH_CACHE=1 policy, 0: its default                  */
    uint32_t entries;      /* graphs retained at most                                                          */
    uint64_t nodes;        /* graph nodes retained at most (bounded)                                           */
    uint32_t sightings;    /* keys tracked before their capture (bounded)                                      */
    uint32_t after;        /* capture at the after-th sighting of a key                                        */
} glmflash_graph_policy;
typedef struct glmflash_graph_stats {
    uint64_t hits, eager, captures, evictions, oversized, retained_graphs, retained_nodes, peak_graphs, peak_nodes,
             largest_graph_nodes, tracked_sightings;
} glmflash_graph_stats;
enum { GLMFLASH_GRAPH_REPLAY = 0, GLMFLASH_GRAPH_EAGER = 1, GLMFLASH_GRAPH_CAPTURE = 2 };
typedef struct glmflash_graph_cache glmflash_graph_cache;
typedef int (*glmflash_enqueue_fn)(void *user, void *stream);
int   glmflash_graph_policy_default(int bounded, glmflash_graph_policy *out);
int   glmflash_graph_cache_new(const glmflash_graph_policy *policy, glmflash_graph_cache **out);
void  glmflash_graph_cache_free(glmflash_graph_cache *c);
int   glmflash_graph_cache_action(glmflash_graph_cache *c, uint64_t key);                 /* GLMFLASH_GRAPH_* or -1 */
int   glmflash_graph_cache_insert(glmflash_graph_cache *c, uint64_t key, uint64_t nodes, void *graph_exec);
void *glmflash_graph_cache_get(const glmflash_graph_cache *c, uint64_t key);              /* cudaGraphExec_t or NULL */
int   glmflash_graph_cache_stats(const glmflash_graph_cache *c, glmflash_graph_stats *out);
/* One window: replay, run eagerly or capture + launch + retain, as the policy decides.  `enqueue` puts the window's
 * work on the stream it is given (any sequence of this library's run calls qualifies) and returns 0 or -1. */
int   glmflash_graph_cache_run(glmflash_graph_cache *c, uint64_t key, void *stream, glmflash_enqueue_fn enqueue, void *user);

#ifdef __cplusplus
}
#endif
#endif /* GLMFLASH_B200_H */
