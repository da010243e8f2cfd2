/* C-ABI of the CUDA (sm_100a) backend for the Clef-Omni mixture-of-experts block.
 *
 * This header is the drop-in boundary: it mirrors the entry points that the reference's
 * shared Metal backend calls on its Omni module (clef_metal_internal.h:65-81, implemented in
 * clef_metal_omni.m) for the MoE half of a decoder layer.  Objective-C handles
 * (id<MTLCommandBuffer>, id<MTLComputeCommandEncoder>) become a CUDA stream owned by the
 * context; everything else keeps the reference's names, argument meaning and error style:
 * every fallible call returns bool and writes a NUL-terminated message into err[errlen].
 *
 * Threading: like the reference (clef_engine.h:152-155) a context is driven by one thread.
 * All device pointers passed in must belong to the context's device.
 */
#ifndef CLEF_CUDA_OMNI_H
#define CLEF_CUDA_OMNI_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque backend state: the CUDA counterpart of `struct clef_gpu`
 * (clef_metal_internal.h:12-57) restricted to what the MoE path needs. */
typedef struct clef_gpu clef_gpu;

/* The fields of clef_config (clef_engine.h:18-33) this path reads. */
typedef struct {
    int n_layer;        /* decoder layers whose expert weights may be bound (<= 128) */
    int H;              /* hidden width: 2048 */
    int ffn;            /* expert intermediate width: 768 */
    int n_expert;       /* 128 */
    int n_expert_used;  /* 8 */
} clef_omni_config;

enum { CLEF_OMNI_HOST = 0, CLEF_OMNI_DEVICE = 1 };

/* Geometry the kernels are compiled for (clef.c:83-93 pins the same numbers). */
enum { CLEF_OMNI_H = 2048, CLEF_OMNI_F = 768, CLEF_OMNI_E = 128, CLEF_OMNI_TOP = 8,
       CLEF_OMNI_CHUNK = 16384 /* tokens per arena pass; longer calls are split */ };

/* ---- lifecycle -------------------------------------------------------------------- */

/* Counterpart of clef_gpu_open (clef_engine.h:165; clef_metal.m:113) for this path: selects
 * `device`, adopts `stream` (a cudaStream_t; NULL creates a private non-blocking stream)
 * and reads the CLEF_* debug environment (CLEF_DEBUG_POISON, CLEF_PROFILE, CLEF_OMNI_ROUTER_EXACT,
 * CLEF_OMNI_ROUTER_EPS, CLEF_DEBUG_OMNI_ALLOC_FAIL, CLEF_DEBUG_OMNI_LAUNCH_FAIL). */
bool clef_cuda_omni_open(clef_gpu **out, int device, void *stream, char *err, size_t errlen);
/* Counterpart of clef_gpu_close (clef_metal.m:241-247): frees arena, trace and owned weights. */
void clef_cuda_omni_close(clef_gpu *g);

/* clef_omni_reserve (clef_metal_omni.m:40-69): rejects T <= 0 and any geometry other than
 * (2048, 768, 128, 8); idempotent once allocated; atomic -- a failed allocation frees what it
 * made and leaves the previous state ("... (previous buffers kept)").  The arena size does
 * not depend on T. */
bool clef_omni_reserve(clef_gpu *g, const clef_omni_config *c, int T, char *err, size_t errlen);
#ifdef CLEF_ENGINE_H
/* For a caller that holds the reference's own clef_config (clef_engine.h:18-33, included before
 * this header): the call of clef_metal.m:1148 with the same arguments. */
static inline bool clef_omni_reserve_config(clef_gpu *g, const clef_config *c, int T, char *err, size_t errlen) {
    clef_omni_config o = {0, 0, 0, 0, 0};
    if (c) { o.n_layer = c->n_layer; o.H = c->H; o.ffn = c->ffn; o.n_expert = c->n_expert; o.n_expert_used = c->n_expert_used; }
    return clef_omni_reserve(g, c ? &o : (const clef_omni_config *)0, T, err, errlen);
}
#endif
/* clef_omni_free (clef_metal_omni.m:71-74). */
void clef_omni_free(clef_gpu *g);
/* clef_omni_begin (clef_metal_omni.m:149-159): clears the status word; with debug poison on,
 * fills every float scratch buffer with NaN. */
void clef_omni_begin(clef_gpu *g);
/* clef_omni_complete (clef_metal_omni.m:161-167): waits for the stream, then reports a
 * nonzero status word as an error.  Bit 0: nonfinite router values (clef.metal:2364).
 * Bit 3: an expert id outside [0,128) reached the permutation.  Bit 4: a bounded device-side
 * wait ran out.  Bit 5: more rows were routed to one rank than its buffers hold (expert
 * parallel only).  Bit 8: the exact router pass met a tensor-core logit further from its exact
 * value than the assumed bound (CLEF_OMNI_ROUTER_EPS, scaled by the row's largest |logit| / 4
 * when that exceeds 1), so rows it did not re-decide cannot be trusted.  A failed launch or
 * stream error is reported here too. */
bool clef_omni_complete(clef_gpu *g, char *err, size_t errlen);
/* clef_omni_keepalive (clef_metal_omni.m:138-147): read-only touch of every arena buffer. */
void clef_omni_keepalive(clef_gpu *g);

/* clef_omni_trace_reserve (clef_metal_omni.m:76-96): enabled=false drops the capture; a
 * failed allocation keeps the previous capture.  Captures the last `rows` rows (0 = all T)
 * of every layer. */
bool clef_omni_trace_reserve(clef_gpu *g, int T, int layers, int rows, bool enabled, char *err, size_t errlen);
/* clef_gpu_dump_routes (clef_metal_omni.m:98-136): validates, then writes one JSON line per
 * (layer, token): logits[128] (%.17g), ids[8], weights[8] (%.9g), margin = 8th - 9th logit.
 * A logit is printed as hi + low: the tensor-core value with low = 0, or, for every logit the
 * exact pass evaluated, its FP64 value as a float pair -- so the ids of a row always follow from
 * the row's printed logits (tests/test_omni_routes.py:28-30). */
bool clef_gpu_dump_routes(clef_gpu *g, const char *path, char *err, size_t errlen);

/* ---- weights ---------------------------------------------------------------------- */

/* Binds one layer's tensors in the converted layout that bind_experts checks
 * (clef.c:194-203, 239-246; tools/convert_omni.py:135-139), all BF16, K contiguous:
 *   router  [128][2048]          (blk.N.ffn_router.weight)
 *   gate_up [128][1536][2048]    (blk.N.ffn_gate_up_exps.weight; gate rows, then up rows)
 *   down    [128][2048][768]     (blk.N.ffn_down_exps.weight)
 * where == CLEF_OMNI_HOST: pointers into host memory (e.g. the mmap'd GGUF); the backend
 * uploads and owns a device copy.  where == CLEF_OMNI_DEVICE: device pointers, borrowed
 * (256-byte aligned).  router_bias (FP32 [128], same location, may be NULL) is an additive
 * logit term; the reference has none. */
bool clef_omni_bind_layer(clef_gpu *g, int layer, const void *router, const void *gate_up, const void *down,
                          const float *router_bias, int where, char *err, size_t errlen);

/* ---- the hot path ----------------------------------------------------------------- */

/* MoE half of clef_omni_encode_layer (clef_metal_omni.m:256-329): reads the normed hidden
 * state `xn` (device, BF16 [T][2048]), adds the routed-expert output into the FP32 residual
 * `x` (device, [T][2048]).  Asynchronous on the context's stream: it only enqueues; errors
 * surface at clef_omni_complete.  seq_bounds (host, n_seq+1 ascending offsets ending at T)
 * is validated; results do not depend on how tokens are grouped into records. */
bool clef_omni_encode_moe(clef_gpu *g, int layer, const void *xn, float *x, int T, int n_seq,
                          const int32_t *seq_bounds, char *err, size_t errlen);

/* One synchronous pass with HOST buffers: begin, copy xn (BF16) and x (FP32) to the device,
 * encode_moe, copy x back, complete.  This is the call a host engine makes when its
 * activations live in host memory.  Above 1536 tokens (one GPU) the batch is processed in
 * pieces of about 1400 tokens whose uploads, kernels and downloads overlap; the bits are
 * those of one pass.  Page-locked host buffers are needed for the copies to overlap. */
bool clef_omni_forward_host(clef_gpu *g, int layer, const void *xn_host, float *x_host, int T, int n_seq,
                            const int32_t *seq_bounds, char *err, size_t errlen);

/* ---- the steps either side of the block ------------------------------------------------- */

/* RMSNorm weights of the layer's `ffn_norm` (FP32 [2048]; clef_engine.h:35-40, bound from
 * `blk.N.ffn_norm.weight`, clef.c:236) and the epsilon of clef_config (clef.c:55).  where as in
 * clef_omni_bind_layer; the library keeps its own device copy.  Atomic like the other binds. */
bool clef_omni_bind_norm(clef_gpu *g, int layer, const float *weight, float eps, int where, char *err, size_t errlen);

/* The reference's sequence `norm(ffn_norm)` + MoE section (clef_metal_omni.m:243 then 256-329) on
 * the FP32 residual stream: xn = BF16(x * rsqrt(mean(x^2) + eps) * w) per token (clef.metal:190-204),
 * then x += MoE(xn).  x is device FP32 [T][2048]; needs clef_omni_bind_norm for the layer. */
bool clef_omni_encode_norm_moe(clef_gpu *g, int layer, float *x, int T, int n_seq, const int32_t *seq_bounds,
                               char *err, size_t errlen);

/* The attention half in front of it: clef_omni_encode_attention (clef_metal_omni.m:200-246), the
 * sequence norm(attn_norm) -> q|k|v projection -> omni_attn_prep (per-head RMS norm of q and k,
 * interleaved three-axis rotary; clef.metal:2073-2130) -> omni_attention (causal inside each record
 * of the packed batch, 32 query heads over 4 key/value heads of 128; clef.metal:2174-2319) -> output
 * projection added into the residual.  The reference's closing norm(ffn_norm) is the first step of
 * clef_omni_encode_norm_moe.  Tensors of one layer, in the converted layout (clef_engine.h:35-40):
 *   attn_norm  FP32 [2048]            (blk.N.attn_norm.weight)
 *   attn_qkv   BF16 [5120][2048]      (blk.N.attn_qkv.weight: 4096 query rows, 512 key rows, 512 value rows)
 *   attn_output BF16 [2048][4096]     (blk.N.attn_output.weight)
 *   q_norm, k_norm FP32 [128]         (blk.N.attn_q_norm / attn_k_norm.weight)
 * eps and rope_theta are clef_config's (1e-6 and 1e6 for Clef-Omni, clef.c:84-86).  where as in
 * clef_omni_bind_layer; the library keeps its own device copy.  The first binding allocates the
 * scratch of the attention half (0.6 GB, independent of T). */
bool clef_omni_bind_attention(clef_gpu *g, int layer, const float *attn_norm, const void *attn_qkv, const void *attn_output,
                              const float *q_norm, const float *k_norm, float eps, float rope_theta, int where, char *err,
                              size_t errlen);
/* x (device FP32 [T][2048], the residual stream) += attention half of `layer`.  pos3: device int32
 * [T][3], each token's temporal, row and column rotary position (clef_record_positions; all three
 * equal to the index inside the record for text).  seq_bounds: host, n_seq + 1 ascending offsets
 * ending at T; a token attends to the earlier tokens of its own record.  T <= 16384 per call, and
 * the record lengths, each rounded up to a multiple of 64, must sum to at most 32768 (a batch of
 * more than 256 records shorter than 64 tokens can exceed that and is refused with a message).
 * Asynchronous like clef_omni_encode_moe; nonfinite q/k/v set status bit 1 (value 2) as in the
 * reference (clef.metal:2120) and fail clef_omni_complete.  BF16 operands on the tensor cores,
 * FP32 softmax and accumulation. */
bool clef_omni_encode_attention(clef_gpu *g, int layer, float *x, const int32_t *pos3, int T, int n_seq,
                                const int32_t *seq_bounds, char *err, size_t errlen);
/* One decoder layer in one call, the drop-in for clef_omni_encode_layer (clef_metal_omni.m:248-331):
 * clef_omni_encode_attention followed by clef_omni_encode_norm_moe on the same residual stream,
 * with the same arguments, limits and error behaviour as those two (the layer needs its attention
 * tensors, its ffn_norm and its expert tensors bound). */
bool clef_omni_encode_layer(clef_gpu *g, int layer, float *x, const int32_t *pos3, int T, int n_seq, const int32_t *seq_bounds,
                            char *err, size_t errlen);

/* Binds layers 0..n_layer-1 from a converted checkpoint (GGUF v3 as tools/convert_omni.py:135-139
 * writes it): router, gate/up and down expert tensors and the ffn_norm weights, with the type,
 * rank and extent checks and messages of clef.c:194-246 (`bind_experts`, `bind_weights`), after the
 * metadata checks of clef.c:27-90 for the keys the block depends on (architecture, layer count,
 * width, intermediate size, expert counts, renormalised top-k, epsilon).  The
 * file is mapped, uploaded and unmapped; with expert parallelism connected, only this rank's
 * experts are uploaded. */
bool clef_omni_bind_gguf(clef_gpu *g, const char *path, int n_layer, char *err, size_t errlen);
/* The same checks without a GPU, for any extents; returns the file's RMS epsilon in *rms_eps. */
bool clef_omni_gguf_check(const char *path, int n_layer, int H, int ffn, int n_expert, float *rms_eps, char *err,
                          size_t errlen);

/* ---- expert parallelism over the GPUs of one node (no counterpart in the reference, which
 *      is single-device; defined by the 1/2/4/8-GPU configurations) -------------------- */

/* The 128 experts are sharded in contiguous ranges of 128/world per rank; tokens stay with the
 * rank that owns them.  Rows travel by peer stores into buffers each rank exports to the others
 * (CUDA IPC between processes, direct peer access inside one process), written by the expert
 * kernels themselves while they compute.  One context per GPU takes part: the kernels of a pass
 * wait for rows from the other ranks, so two contexts of one GPU could wait on each other.  Order of calls on
 * every rank: open, reserve, ep_export, [exchange handles], ep_connect, bind_layer, then
 * begin / encode_moe / complete as usual; every rank must make the same sequence of encode_moe
 * calls (T <= 16384 per call, T may differ per rank).  After connect:
 *   - bind_layer with CLEF_OMNI_HOST uploads only the rank's expert slice (router in full);
 *     with CLEF_OMNI_DEVICE gate_up/down must already be the rank's slice
 *     [128/world][1536][2048] and [128/world][2048][768].
 *   - results are bitwise those of the single-GPU path on the same tokens. */
typedef struct { unsigned char reserved[64]; } clef_omni_ipc_handle;
enum { CLEF_OMNI_EP_HANDLES = 6, CLEF_OMNI_EP_MAX_WORLD = 8 };
bool clef_omni_ep_export(clef_gpu *g, clef_omni_ipc_handle out[CLEF_OMNI_EP_HANDLES], char *err, size_t errlen);
/* all = world x CLEF_OMNI_EP_HANDLES handles, rank-major, as exported by every rank */
bool clef_omni_ep_connect(clef_gpu *g, int rank, int world, const clef_omni_ipc_handle *all, char *err, size_t errlen);
/* same, for contexts that live in one process: peers[r] is rank r's context */
bool clef_omni_ep_connect_local(clef_gpu *g, int rank, int world, clef_gpu *const *peers, char *err, size_t errlen);
void clef_omni_ep_disconnect(clef_gpu *g);
/* One barrier across the ranks on the context's stream, waited for on the host (timeout_ms <= 0:
 * 2 s).  Every rank calls it once after all ranks have connected (it also makes the first, slow
 * touch of the peers' memory happen here and not in the first pass).  It is also how ranks get
 * back in step: the ranks agree on a common barrier epoch here, whatever each one's was.  A
 * pass that fails on one rank (a refused launch, a wait on the others that ran out) leaves that
 * rank's context refusing further passes until this call has succeeded on every rank; a rank
 * that waited alone may simply call again.  Inside a pass every wait on another rank is bounded
 * (2 s, or option "ep_wait_ms"); ranks that start a pass further apart than that fail the pass
 * with status bit 4.  Capacity: a pass is refused (status bit 5, on every rank) when more than
 * 131072 expert rows from all ranks together are routed to the experts of one rank -- with
 * evenly spread routing that is 16384 tokens per rank, with skewed routing fewer. */
bool clef_omni_ep_sync(clef_gpu *g, int timeout_ms, char *err, size_t errlen);
/* ---- stage entry points (model-free tests, mirroring tests/test_omni_*.m) ---------- */

/* omni_router (clef.metal:2330-2345): logits[t][e] as FP64 sums of exact BF16 products. */
bool clef_omni_stage_router(clef_gpu *g, int layer, const void *xn, int T, double *logits, char *err, size_t errlen);
/* omni_route (clef.metal:2347-2394) on given hi/lo logit pairs (lo may be NULL): ids
 * descending by hi+lo, ties to the lowest id; weights renormalised over the selected. */
bool clef_omni_stage_route(clef_gpu *g, const float *hi, const float *lo, int rows, int32_t *ids, float *weights,
                           char *err, size_t errlen);
/* omni_assign_count/offsets/scatter (clef.metal:2396-2443) in canonical form: counts[128],
 * offsets[129] = exclusive prefix sum of counts, rowmap[rows*8] = token of each permuted
 * row, slots[rows*8] = permuted row of assignment t*8+k.  Stable. */
bool clef_omni_stage_assign(clef_gpu *g, const int32_t *ids, int rows, int32_t *counts, int32_t *offsets,
                            int32_t *rowmap, int32_t *slots, char *err, size_t errlen);
/* gather + expert products + combine (clef.metal:2445-2523) with routing supplied by the
 * caller: x[t] += sum_k weights[t][k] * expert_{ids[t][k]}(xn[t]). */
bool clef_omni_stage_experts(clef_gpu *g, int layer, const void *xn, const int32_t *ids, const float *weights,
                             float *x, int T, char *err, size_t errlen);

/* ---- a call that never allocates --------------------------------------------------- */

/* No counterpart in the reference.  Some hosts cannot take a device allocation on their hot
 * path at all: code that runs while a CUDA stream is being captured, a real-time loop that
 * must not touch the driver's allocator, a plug-in that is handed a fixed memory budget and
 * no context of its own.  Every other entry point here works on a context whose arena comes
 * from cudaMalloc.  This one needs no context: it is the stable counting sort of
 * clef_omni_stage_assign (same inputs, same outputs, same bits) with its scratch -- segment
 * histograms, tile list, counters, about 72 KB -- in a fixed device array that is part of the
 * library image, so every GPU that loads the library carries it until the process exits.
 *   - at most CLEF_OMNI_NOALLOC_MAX_ROWS tokens per call; more is refused with a message;
 *   - ids, counts[128], offsets[129], rowmap[rows*8], slots[rows*8] are device pointers on the
 *     current device; status (device, one word) receives bit 3 when an expert id is out of
 *     range, as in clef_omni_complete; the caller clears it.  status may be NULL, but then
 *     nothing reports such an id: it is sorted as id & 127 and the call still returns true;
 *   - work is enqueued on `stream` (a cudaStream_t, NULL = default stream); nothing is waited for;
 *   - the first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress); make that first call outside any stream capture;
 *   - all calls on a device share the one array: calls that may overlap on the GPU (different
 *     streams, no ordering between them) race on it.  Nothing in it has to be zero on entry. */
enum { CLEF_OMNI_NOALLOC_MAX_ROWS = 4096 };
bool clef_omni_assign_noalloc(const int32_t *ids, int rows, int32_t *counts, int32_t *offsets, int32_t *rowmap,
                              int32_t *slots, uint32_t *status, void *stream, char *err, size_t errlen);

/* ---- introspection, options, profiling -------------------------------------------- */

/* Copies an arena buffer of the last pass to host memory after waiting for the stream:
 * "ids" int32[T][8], "weights" f32[T][8], "logits" f32[T][128], "counts" int32[128],
 * "offsets" int32[129], "rowmap" int32[T*8], "slots" int32[T*8], "status" u32,
 * "rechecked" int32 (rows whose order was decided by the exact pass), "xnorm" bf16[T][2048]
 * (the normalised rows clef_omni_encode_norm_moe fed to the block); of the last attention pass:
 * "attn_qkv" bf16 [T][5120] (the q|k|v projections) and "attn_out" bf16 [T][4096] (the attention
 * output before the output projection). */
bool clef_omni_read(clef_gpu *g, const char *what, void *dst, size_t bytes, char *err, size_t errlen);
/* Options: "debug_poison" 0/1 (CLEF_DEBUG_POISON), "router_exact" 0/1 (decide every row with
 * FP64 logits), "router_eps" (bound on the tensor-core logit error, x1e-9), "gemm" 0 =
 * tcgen05 kernels, 1 = plain CUDA-core check kernels, "router" likewise, "profile" 0/1,
 * "ep_fused" 0/1 (expert parallelism, default 1: the expert kernels move the rows themselves -- the
 * gate/up kernel's spare warps send the token rows while it computes, the down kernel writes its
 * results straight to the ranks they belong to; 0: a copy kernel and a barrier in front of the
 * gate/up kernel; same results; must be the same on every rank, as it changes the number of barriers per pass),
 * "expert_kernel" 0/1/2 (2: expert products on pairs of CTAs, tcgen05.mma.cta_group::2; 1: the same
 * kernel on single CTAs; 0: the earlier single-CTA kernels; same results),
 * "longest_first" 0/1 (default 1: the gate/up kernel claims its work items in order of falling tile length, the
 * short ones filling the end of the launch; 0: in expert order; same results; set after clef_omni_reserve),
 * "expert_chain" 0/1 (default 0; one GPU, single-CTA kernels: the down kernel does not wait for the
 * whole gate/up grid but starts on the SMs its first blocks leave and takes each expert's rows once
 * a per-expert counter says they are complete; same results; about 1 % faster while the GPU is
 * cool, nothing once the power limit sets the clock),
 * "ep_wait_ms" N (bound on each in-pass wait for other ranks, 0 = 2000), "reserve_sms" N (the persistent expert kernels use all SMs but N, so that kernels of another
 * context on the same GPU -- another micro-batch -- are not locked out while they run),
 * "fused_gather" 0/1 (default 1: the gate/up kernel fetches its token rows through the permutation
 * itself instead of reading a copy in expert order made by a separate kernel; same results),
 * "fused_router" 0/1 (default 1: the router kernel counts the experts per segment of the counting sort,
 * so no histogram kernel runs; same results),
 * "dependent_launch" 0/1 (default 1, process-wide: the kernels of a pass are launched so that each one's
 * prologue overlaps the tail of the one before),
 * "alloc_fail_at" N / "launch_fail_at" N (host-side fault injection, 0 = off). */
bool clef_omni_set_option(clef_gpu *g, const char *name, long value);
/* With "profile" on every pass records stage marks on the stream without waiting.  This call
 * waits for the stream and returns the mean device milliseconds per pass over the passes
 * recorded since the previous call (at most the last 64), in the order router, permute
 * (histogram + sort + gather), gate_up, down, combine, total; then restarts the count. */
bool clef_omni_profile(clef_gpu *g, float ms[6]);
/* Arena bytes currently reserved (0 when not reserved). */
size_t clef_omni_arena_bytes(const clef_gpu *g);

#ifdef __cplusplus
}
#endif
#endif
