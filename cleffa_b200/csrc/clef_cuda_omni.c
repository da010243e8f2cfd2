/* CUDA backend for the Clef-Omni mixture-of-experts block: host side.
 *
 * Mirrors the Omni module of the reference's Metal backend (clef_metal_omni.m): a scratch
 * arena with an atomic reserve, a device status word cleared by begin and checked by complete,
 * per-chunk stage dispatch, optional route capture with a JSONL dump.  A command buffer
 * becomes a CUDA stream; "encode" only enqueues work and errors surface at completion, as in
 * the reference (clef_metal.m:1591-1597).
 *
 * There is no CPU fallback: every stage is a CUDA kernel (omni_kernels.cu, omni_sm100.cu).
 */
#define _GNU_SOURCE
#include "clef_cuda_omni.h"
#include "omni_internal.h"

#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

enum { MAX_LAYERS = 128, N_STAGE_EVENTS = 6, PROF_SLOTS = 64, HOST_PIECES = 16 };

/* Route capture row, byte-compatible with omni_route_row (clef_metal_omni.m:15): 1088 bytes. */
typedef struct { float logits[OMNI_E], low[OMNI_E]; int32_t ids[OMNI_TOP]; float weights[OMNI_TOP]; } omni_route_row;

typedef struct {
    void *router, *gate_up, *down;      /* device, BF16 */
    float *bias;                        /* device, FP32 [128] or NULL */
    bool owned, bound;
    CUtensorMap tm_router, tm_gate_up, tm_down;
    CUtensorMap tm_gate_up3;            /* {K, gate|up, row} view of gate_up: a box interleaves gate and up rows */
} omni_layer;

/* The scratch arena (clef_omni_gpu in the reference, clef_metal_omni.m:18-23). */
typedef struct {
    float *logits;                      /* [CHUNK][128] router logits: tensor-core values, exact (hi) where the exact pass ran */
    float *logits_low;                  /* [CHUNK][128] remainder of the exact logits (hi + low); zero elsewhere; kept for route capture */
    int32_t *ids; float *weights;       /* [CHUNK][8] */
    int32_t *flag_rows, *n_flag;        /* rows handed to the exact pass */
    uint32_t *status, *sink;
    unsigned long long *stamps;         /* [CHUNK/128][8] optional router timestamps */
    omni_sort_state sort;
    void *xg, *h, *d;                   /* permuted rows: BF16 [ROWS][2048], [ROWS][768], [ROWS][2048] */
    CUtensorMap tm_xg[4], tm_h[4];      /* box heights 32, 64, 128, 256 rows */
    size_t bytes;
} omni_arena;

struct clef_gpu {
    int device, n_sm;
    cudaStream_t stream;
    bool own_stream;
    omni_arena *omni;
    omni_layer layer[MAX_LAYERS];
    int n_layer;
    /* RMSNorm in front of the block (clef_omni_bind_norm / clef_omni_encode_norm_moe) */
    float *norm_w[MAX_LAYERS];          /* device, FP32 [2048]; NULL = not bound */
    float norm_eps[MAX_LAYERS];
    void *xnorm;                        /* BF16 [CHUNK][2048]: the normalised rows of the chunk in flight */
    /* attention half (clef_omni_bind_attention / clef_omni_encode_attention) */
    struct {
        float *norm_w, *q_norm, *k_norm;   /* device FP32 [2048], [128], [128] */
        void *qkv, *out;                   /* device BF16 [5120][2048], [2048][4096] */
        float eps; double theta;
        bool bound;
        CUtensorMap tm_qkv, tm_out;
    } attn[MAX_LAYERS];
    struct {
        void *p, *q, *k, *vt, *a;          /* BF16: q|k|v rows [CHUNK][5120]; Q [32][CHUNK][128]; K [4][CHUNK][128]; Vt [4][128][VPITCH]; attention output [CHUNK][4096] */
        int32_t *tiles, *vcol, *sched;     /* device: query tiles, Vt column of every token, work counters of the two projections */
        int32_t *h_tiles, *h_vcol, *h_bounds;   /* host copies; h_bounds remembers the batch the device copies describe */
        int n_tiles, last_T, last_nseq;
        CUtensorMap tm_xn[4], tm_a[4], tm_q, tm_k, tm_vt;
        bool ready;
    } at;
    /* route capture */
    omni_route_row *trace;              /* device */
    int trace_first, trace_rows, trace_layers;
    bool trace_valid;
    /* options */
    bool debug_poison, router_exact, profile, debug_stamps;
    int ep_fused;                       /* expert parallelism: the expert kernels move the rows themselves (default 1) */
    float router_eps;
    int gemm_impl, router_impl;         /* 0 = tcgen05, 1 = CUDA-core check kernels */
    int expert_chain;                   /* 1: on one GPU the down kernel is chained behind gate/up per expert (default 0: worth ~1 % only while the GPU is cool) */
    int expert_kernel;                  /* tcgen05 expert products: 2 = pairs of CTAs (cta_group::2), 1 = the same kernel on
                                           single CTAs, 0 = the earlier single-CTA kernels (two accumulators for gate/up) */
    int reserve_sms;                    /* SMs the persistent expert kernels leave to other streams */
    int host_pieces;                    /* clef_omni_forward_host: pieces the batch is cut into (0 = chosen from T) */
    int fused_router;                   /* the router kernel counts experts per sort segment (no histogram kernel) */
    int fused_gather;                   /* gate/up fetches its token rows through rowmap (no gather kernel) */
    long alloc_fail_at, alloc_count;    /* host-side fault injection */
    long launch_fail_at, launch_count;
    /* pass state */
    bool failed;                        /* a launch or copy of this pass failed (cb_failed, clef_metal_internal.h:52) */
    char fail_msg[160];
    int last_T;
    cudaEvent_t ev[PROF_SLOTS][N_STAGE_EVENTS];   /* ring of per-pass stage marks, read by clef_omni_profile */
    long prof_passes;
    void *stage_x, *stage_res;          /* forward_host staging */
    size_t stage_cap;
    /* forward_host: uploads, kernels and downloads of successive pieces of the batch overlap */
    cudaStream_t copy_stream, out_stream;
    cudaEvent_t ev_xn[HOST_PIECES], ev_res[HOST_PIECES], ev_done[HOST_PIECES];
    cudaEvent_t residual_uploaded;      /* the ev_res[] entry of the piece being encoded */
    bool wait_residual;                 /* the combine of the current pass must wait for that upload */
    /* expert parallelism (omni_ep.cu); world <= 1 means off */
    struct {
        int rank, world;
        bool ipc;                        /* peers opened through CUDA IPC (else direct pointers) */
        omni_ep_peers peers;
        uint32_t epoch;                  /* last barrier epoch this rank launched */
        uint32_t sync_count;             /* successful clef_omni_ep_sync calls, as agreed between the ranks */
        bool need_sync;                  /* a pass failed: the ranks may be out of step until the next sync */
        uint64_t wait_ns;                /* bound on every in-pass wait for other ranks; 0 = 2 s */
        uint32_t *sync_result;           /* device [2] */
        void *dret; int32_t *rowinfo, *counts, *send_base, *n_local_rows; uint32_t *flags;
        void *opened[OMNI_EP_MAX][OMNI_EP_BUFFERS];
        int32_t *need;                        /* [128] rows each group of local experts must receive */
        /* de-duplicated dispatch: token -> (owner, group) buckets and where they land on the owners */
        int32_t *tok_slot, *bucket_cnt, *bucket_list, *send_cnt, *recv_base, *grow;
    } ep;
    CUresult (*encode_tiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                             const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                             CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
};

static void set_err(char *err, size_t errlen, const char *fmt, ...) {
    if (!err || !errlen) return;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err, errlen, fmt, ap);
    va_end(ap);
}

static void note_failure(clef_gpu *g, const char *what, cudaError_t e) {
    if (g->failed) return;
    g->failed = true;
    snprintf(g->fail_msg, sizeof g->fail_msg, "cuda: %s failed: %s", what, cudaGetErrorString(e));
}

/* Every stage launch goes through here so a test can make the Nth one fail on the host
 * (the counterpart of CLEF_DEBUG_NIL_CMDBUF, clef_metal_internal.h:53). */
static bool launched(clef_gpu *g, const char *what, cudaError_t e) {
    if (g->launch_fail_at > 0 && ++g->launch_count == g->launch_fail_at) e = cudaErrorLaunchFailure;
    if (e == cudaSuccess) return true;
    note_failure(g, what, e);
    return false;
}

/* ---------------------------------------------------------------- allocation */
static void *dev_alloc(clef_gpu *g, size_t bytes) {
    void *p = NULL;
    if (g->alloc_fail_at > 0 && ++g->alloc_count == g->alloc_fail_at) return NULL;
    if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); return NULL; }
    return p;
}

static bool make_map(clef_gpu *g, CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                     CUtensorMapL2promotion promo) {
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return g->encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)base, dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, promo,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

/* The gate/up matrix of the bound experts, [n_expert][gate rows 0..767 ; up rows 0..767][2048], as a
 * three-dimensional tensor {K, 2, row}: coordinate (k, 0, e*1536 + f) with box {64, 2, 64} brings
 * gate row f+i and up row f+i (i < 64) of expert e into consecutive shared-memory rows 2i, 2i+1. */
static bool make_gate_up3(clef_gpu *g, CUtensorMap *map, const void *base, uint64_t n_expert) {
    const cuuint64_t dims[3] = {OMNI_H, 2, n_expert * 2 * OMNI_F - OMNI_F};
    const cuuint64_t strides[2] = {(cuuint64_t)OMNI_F * OMNI_H * 2, (cuuint64_t)OMNI_H * 2};
    const cuuint32_t box[3] = {64, 2, 64};
    const cuuint32_t estr[3] = {1, 1, 1};
    return g->encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void *)base, dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

/* ---------------------------------------------------------------- lifecycle */
bool clef_cuda_omni_open(clef_gpu **out, int device, void *stream, char *err, size_t errlen) {
    if (!out) { set_err(err, errlen, "cuda: null context pointer"); return false; }
    *out = NULL;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) { set_err(err, errlen, "cuda: cannot select device %d: %s", device, cudaGetErrorString(e)); return false; }
    struct cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) { set_err(err, errlen, "cuda: cannot query device %d: %s", device, cudaGetErrorString(e)); return false; }
    if (prop.major != 10) {
        set_err(err, errlen, "cuda: device %d is sm_%d%d; this backend is built for sm_100a only", device, prop.major, prop.minor);
        return false;
    }
    clef_gpu *g = calloc(1, sizeof *g);
    if (!g) { set_err(err, errlen, "cuda: cannot allocate backend state"); return false; }
    g->device = device;
    g->n_sm = prop.multiProcessorCount;
    g->router_eps = 5e-4f;
    g->fused_gather = 1;
    g->fused_router = 1;
    g->ep_fused = 1;
    g->expert_chain = 0;
    void *fn = NULL;
    enum cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || !fn || qres != cudaDriverEntryPointSuccess) {
        set_err(err, errlen, "cuda: driver lacks cuTensorMapEncodeTiled");
        free(g);
        return false;
    }
    *(void **)&g->encode_tiled = fn;
    if (stream) g->stream = (cudaStream_t)stream;
    else {
        e = cudaStreamCreateWithFlags(&g->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) { set_err(err, errlen, "cuda: cannot create stream: %s", cudaGetErrorString(e)); free(g); return false; }
        g->own_stream = true;
    }
    e = omni_sm100_configure();
    if (e == cudaSuccess) e = omni_expert_configure();
    if (e == cudaSuccess) e = omni_router_configure();
    if (e == cudaSuccess) e = omni_attn_configure();
    if (e != cudaSuccess) {
        set_err(err, errlen, "cuda: cannot configure sm_100a kernels: %s", cudaGetErrorString(e));
        if (g->own_stream) cudaStreamDestroy(g->stream);
        free(g);
        return false;
    }
    for (int p = 0; p < PROF_SLOTS && e == cudaSuccess; p++)
        for (int i = 0; i < N_STAGE_EVENTS && e == cudaSuccess; i++) e = cudaEventCreate(&g->ev[p][i]);
    if (e != cudaSuccess) {
        set_err(err, errlen, "cuda: cannot create the stage events: %s", cudaGetErrorString(e));
        cudaGetLastError();
        clef_cuda_omni_close(g);
        return false;
    }
    const char *v;
    if ((v = getenv("CLEF_DEBUG_POISON")) && *v == '1') g->debug_poison = true;
    if ((v = getenv("CLEF_PROFILE")) && *v == '1') g->profile = true;
    if ((v = getenv("CLEF_OMNI_ROUTER_EXACT")) && *v == '1') g->router_exact = true;
    if ((v = getenv("CLEF_OMNI_ROUTER_EPS"))) { float f = strtof(v, NULL); if (f > 0 && isfinite(f)) g->router_eps = f; }
    if ((v = getenv("CLEF_DEBUG_OMNI_ALLOC_FAIL"))) g->alloc_fail_at = strtol(v, NULL, 10);
    if ((v = getenv("CLEF_DEBUG_OMNI_LAUNCH_FAIL"))) g->launch_fail_at = strtol(v, NULL, 10);
    *out = g;
    return true;
}

void clef_omni_ep_disconnect(clef_gpu *g);
static void attn_free(clef_gpu *g);

static void free_layer(omni_layer *L) {
    if (L->owned) { cudaFree(L->router); cudaFree(L->gate_up); cudaFree(L->down); cudaFree(L->bias); }
    memset(L, 0, sizeof *L);
}

static void free_arena(omni_arena *s) {
    if (!s) return;
    void *all[] = {s->logits, s->logits_low, s->ids, s->weights, s->flag_rows, s->n_flag, s->status, s->sink, s->sort.counts,
                   s->sort.offsets, s->sort.rowmap, s->sort.slots, s->sort.segcount, s->sort.ttiles, s->sort.n_ttiles, s->sort.sched,
                   s->xg, s->h, s->d, s->stamps};
    for (size_t i = 0; i < sizeof all / sizeof all[0]; i++) if (all[i]) cudaFree(all[i]);
    free(s);
}

void clef_omni_free(clef_gpu *g) {
    if (!g) return;
    clef_omni_ep_disconnect(g);          /* the exchange buffers include the arena's */
    free_arena(g->omni);
    g->omni = NULL;
}

void clef_cuda_omni_close(clef_gpu *g) {
    if (!g) return;
    cudaSetDevice(g->device);
    cudaStreamSynchronize(g->stream);
    clef_omni_ep_disconnect(g);
    clef_omni_free(g);
    for (int l = 0; l < MAX_LAYERS; l++) free_layer(&g->layer[l]);
    attn_free(g);
    for (int l = 0; l < MAX_LAYERS; l++) if (g->norm_w[l]) cudaFree(g->norm_w[l]);
    if (g->xnorm) cudaFree(g->xnorm);
    if (g->trace) cudaFree(g->trace);
    if (g->stage_x) cudaFree(g->stage_x);
    if (g->stage_res) cudaFree(g->stage_res);
    if (g->copy_stream) { cudaStreamSynchronize(g->copy_stream); cudaStreamDestroy(g->copy_stream); }
    if (g->out_stream) { cudaStreamSynchronize(g->out_stream); cudaStreamDestroy(g->out_stream); }
    for (int i = 0; i < HOST_PIECES; i++) {
        if (g->ev_xn[i]) cudaEventDestroy(g->ev_xn[i]);
        if (g->ev_res[i]) cudaEventDestroy(g->ev_res[i]);
        if (g->ev_done[i]) cudaEventDestroy(g->ev_done[i]);
    }
    for (int p = 0; p < PROF_SLOTS; p++) for (int i = 0; i < N_STAGE_EVENTS; i++) if (g->ev[p][i]) cudaEventDestroy(g->ev[p][i]);
    if (g->own_stream) cudaStreamDestroy(g->stream);
    free(g);
}

bool clef_omni_reserve(clef_gpu *g, const clef_omni_config *c, int T, char *err, size_t errlen) {
    if (!g || !c || T <= 0 || c->H != OMNI_H || c->ffn != OMNI_F || c->n_expert != OMNI_E || c->n_expert_used != OMNI_TOP ||
        c->n_layer <= 0 || c->n_layer > MAX_LAYERS) {
        set_err(err, errlen, "cuda: invalid Omni scratch dimensions");
        return false;
    }
    if (g->omni) { if (c->n_layer > g->n_layer) g->n_layer = c->n_layer; return true; }
    cudaSetDevice(g->device);
    omni_arena *s = calloc(1, sizeof *s);
    if (!s) { set_err(err, errlen, "cuda: cannot allocate Omni state"); return false; }
    struct { void **p; size_t bytes; } want[] = {
        {(void **)&s->logits, (size_t)OMNI_CHUNK * OMNI_E * 4},
        {(void **)&s->logits_low, (size_t)OMNI_CHUNK * OMNI_E * 4},
        {(void **)&s->ids, (size_t)OMNI_CHUNK * OMNI_TOP * 4},
        {(void **)&s->weights, (size_t)OMNI_CHUNK * OMNI_TOP * 4},
        {(void **)&s->flag_rows, (size_t)OMNI_CHUNK * 4},
        {(void **)&s->n_flag, 2048},       /* [0..1] flagged-row counts; from word 64: done[128], done_need[128] */
        {(void **)&s->status, 256},
        {(void **)&s->sink, 256},
        {(void **)&s->stamps, (size_t)(OMNI_CHUNK / 32) * 8 * 8},
        {(void **)&s->sort.counts, (size_t)OMNI_E * 4},
        {(void **)&s->sort.offsets, (size_t)(OMNI_E + 1) * 4},
        {(void **)&s->sort.rowmap, (size_t)OMNI_ROWS * 4},
        {(void **)&s->sort.slots, (size_t)OMNI_ROWS * 4},
        {(void **)&s->sort.segcount, (size_t)OMNI_MAX_SEGS * OMNI_E * 4},
        {(void **)&s->sort.ttiles, (size_t)2 * OMNI_MAX_TTILES * sizeof(omni_ttile)},      /* the list, and the same tiles in expert order */
        {(void **)&s->sort.n_ttiles, 256},
        {(void **)&s->sort.sched, 256},
        {&s->xg, (size_t)OMNI_ROWS * OMNI_H * 2},
        {&s->h, (size_t)OMNI_ROWS * OMNI_F * 2},
        {&s->d, (size_t)OMNI_ROWS * OMNI_H * 2},
    };
    bool ok = true;
    for (size_t i = 0; i < sizeof want / sizeof want[0] && ok; i++) {
        *want[i].p = dev_alloc(g, want[i].bytes);
        if (!*want[i].p) ok = false;
        else s->bytes += want[i].bytes;
    }
    s->sort.status = s->status;
    s->sort.n_flag = s->n_flag;
    s->sort.longest_first = 1;
    s->sort.ttiles_down = ok ? s->sort.ttiles + OMNI_MAX_TTILES : NULL;
    s->sort.done = ok ? s->n_flag + 64 : NULL;
    s->sort.done_need = ok ? s->n_flag + 192 : NULL;
    for (int i = 0; i < 4 && ok; i++)
        ok = make_map(g, &s->tm_xg[i], s->xg, OMNI_ROWS, OMNI_H, 32u << i, CU_TENSOR_MAP_L2_PROMOTION_L2_128B) &&
             make_map(g, &s->tm_h[i], s->h, OMNI_ROWS, OMNI_F, 32u << i, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (ok) ok = cudaMemsetAsync(s->status, 0, 256, g->stream) == cudaSuccess &&
                 cudaMemsetAsync(s->sink, 0, 256, g->stream) == cudaSuccess &&
                 cudaMemsetAsync(s->n_flag, 0, 2048, g->stream) == cudaSuccess &&
                 cudaMemsetAsync(s->sort.n_ttiles, 0, 256, g->stream) == cudaSuccess &&
                 cudaStreamSynchronize(g->stream) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        free_arena(s);
        set_err(err, errlen, "cuda: cannot allocate Omni expert arena (previous buffers kept)");
        return false;
    }
    g->omni = s;
    g->n_layer = c->n_layer;
    return true;
}

size_t clef_omni_arena_bytes(const clef_gpu *g) { return g && g->omni ? g->omni->bytes : 0; }

static void poison(clef_gpu *g, void *p, size_t bytes, uint32_t pattern) {
    launched(g, "poison fill", omni_launch_fill_u32(p, pattern, bytes / 4, g->stream));
}

void clef_omni_begin(clef_gpu *g) {
    if (!g || !g->omni) return;
    omni_arena *s = g->omni;
    cudaSetDevice(g->device);
    g->failed = false;
    g->fail_msg[0] = 0;
    g->trace_valid = false;
    if (cudaMemsetAsync(s->status, 0, 4, g->stream) != cudaSuccess) note_failure(g, "status clear", cudaGetLastError());
    /* a pass that failed between the router and the scan leaves its flagged-row count behind */
    if (cudaMemsetAsync(s->n_flag, 0, 4, g->stream) != cudaSuccess) note_failure(g, "flag clear", cudaGetLastError());
    /* likewise the bucket counters of the expert-parallel dispatch (cleared by the plan kernel in a pass that gets that far) */
    if (g->ep.world > 1 && cudaMemsetAsync(g->ep.bucket_cnt, 0, (size_t)OMNI_EP_BUCKETS * 4, g->stream) != cudaSuccess)
        note_failure(g, "bucket clear", cudaGetLastError());
    if (g->debug_poison) {
        /* clef_metal_omni.m:152-158: every float scratch buffer starts as NaN */
        poison(g, s->logits, (size_t)OMNI_CHUNK * OMNI_E * 4, 0x7fc00000u);
        poison(g, s->weights, (size_t)OMNI_CHUNK * OMNI_TOP * 4, 0x7fc00000u);
        poison(g, s->xg, (size_t)OMNI_ROWS * OMNI_H * 2, 0x7fc07fc0u);
        poison(g, s->h, (size_t)OMNI_ROWS * OMNI_F * 2, 0x7fc07fc0u);
        poison(g, s->d, (size_t)OMNI_ROWS * OMNI_H * 2, 0x7fc07fc0u);
        if (g->trace) poison(g, g->trace, (size_t)g->trace_layers * g->trace_rows * sizeof(omni_route_row), 0x7fc00000u);
    }
}

bool clef_omni_complete(clef_gpu *g, char *err, size_t errlen) {
    if (!g || !g->omni) { set_err(err, errlen, "cuda: Omni arena not reserved"); return false; }
    cudaSetDevice(g->device);
    uint32_t status = 0;
    cudaError_t e = cudaStreamSynchronize(g->stream);
    if (e == cudaSuccess) e = cudaMemcpy(&status, g->omni->status, 4, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { set_err(err, errlen, "cuda: Omni pass failed: %s", cudaGetErrorString(e)); return false; }
    if (g->failed) { set_err(err, errlen, "%s", g->fail_msg); return false; }
    if (status & OMNI_ST_TIMEOUT) {
        if (g->ep.world > 1) g->ep.need_sync = true;
        set_err(err, errlen, "cuda: a bounded device wait ran out in an Omni expert kernel (%s, status 0x%x)",
                status & OMNI_ST_TIMEOUT_BARRIER ? "barrier between ranks" :
                status & OMNI_ST_TIMEOUT_ARRIVAL ? "rows from other ranks did not arrive" : "pipeline barrier", status);
        return false;
    }
    if (status & OMNI_ST_EP_OVERFLOW) { set_err(err, errlen, "cuda: more expert rows were routed to this rank than its Omni arena holds"); return false; }
    if (status & OMNI_ST_BAD_ID) { set_err(err, errlen, "cuda: expert id outside [0,128) reached the Omni permutation"); return false; }
    if (status & OMNI_ST_ROUTER_EPS) {
        set_err(err, errlen, "cuda: router accumulation error exceeded CLEF_OMNI_ROUTER_EPS (%g): raise it or set CLEF_OMNI_ROUTER_EXACT=1",
                (double)g->router_eps);
        return false;
    }
    if (status) { set_err(err, errlen, "cuda: nonfinite Omni attention or router values"); return false; }
    g->trace_valid = g->trace != NULL;
    return true;
}

void clef_omni_keepalive(clef_gpu *g) {
    if (!g || !g->omni) return;
    omni_arena *s = g->omni;
    cudaSetDevice(g->device);
    const void *buffers[] = {s->logits, s->ids, s->weights, s->status, s->sort.counts, s->sort.offsets, s->sort.rowmap,
                             s->sort.slots, s->xg, s->h, s->d, g->trace};
    for (size_t i = 0; i < sizeof buffers / sizeof buffers[0]; i++)
        if (buffers[i]) omni_launch_touch(buffers[i], NULL, g->stream);
}

/* ---------------------------------------------------------------- route capture */
bool clef_omni_trace_reserve(clef_gpu *g, int T, int layers, int rows, bool enabled, char *err, size_t errlen) {
    if (!g || !g->omni) { set_err(err, errlen, "cuda: Omni arena not reserved"); return false; }
    cudaSetDevice(g->device);
    if (!enabled) {
        cudaStreamSynchronize(g->stream);
        if (g->trace) cudaFree(g->trace);
        g->trace = NULL;
        g->trace_rows = g->trace_layers = 0;
        g->trace_valid = false;
        return true;
    }
    if (T <= 0 || layers <= 0 || layers > MAX_LAYERS || rows < 0) {
        set_err(err, errlen, "cuda: invalid Omni trace dimensions");
        return false;
    }
    const int R = rows > 0 && rows < T ? rows : T;
    omni_route_row *next = dev_alloc(g, (size_t)layers * R * sizeof(omni_route_row));
    if (!next) {
        set_err(err, errlen, "cuda: cannot allocate Omni route capture (previous buffers kept)");
        return false;
    }
    cudaStreamSynchronize(g->stream);
    if (g->trace) cudaFree(g->trace);
    g->trace = next;
    g->trace_first = T - R; g->trace_rows = R; g->trace_layers = layers;
    g->trace_valid = false;
    return true;
}

/* A captured row is usable when every logit pair is finite and every selected id and weight
 * is in range; the file is only created once all rows passed (clef_metal_omni.m:105-113). */
static const char *route_row_defect(const omni_route_row *r) {
    for (int e = 0; e < OMNI_E; e++)
        if (!isfinite(r->logits[e]) || !isfinite(r->low[e])) return "nonfinite captured Omni router logits";
    for (int k = 0; k < OMNI_TOP; k++)
        if (r->ids[k] < 0 || r->ids[k] >= OMNI_E || !isfinite(r->weights[k])) return "invalid captured Omni routes";
    return NULL;
}

/* One JSON line: {"layer","token","logits":[128 x hi+low, %.17g],"ids":[8],"weights":[8 x %.9g],
 * "margin": 8th - 9th highest logit} -- the schema tests/compare_omni_routes.py:37-64 reads. */
static void route_row_print(FILE *f, int layer, int token, const omni_route_row *r) {
    double v[OMNI_E], best[OMNI_TOP + 1];
    bool used[OMNI_E] = {false};
    for (int e = 0; e < OMNI_E; e++) v[e] = (double)r->logits[e] + (double)r->low[e];
    for (int k = 0; k <= OMNI_TOP; k++) {            /* the nine highest values by repeated selection */
        int at = -1;
        for (int e = 0; e < OMNI_E; e++) if (!used[e] && (at < 0 || v[e] > v[at])) at = e;
        used[at] = true;
        best[k] = v[at];
    }
    fprintf(f, "{\"layer\":%d,\"token\":%d,\"logits\":[", layer, token);
    for (int e = 0; e < OMNI_E; e++) fprintf(f, e ? ",%.17g" : "%.17g", v[e]);
    fputs("],\"ids\":[", f);
    for (int k = 0; k < OMNI_TOP; k++) fprintf(f, k ? ",%d" : "%d", r->ids[k]);
    fputs("],\"weights\":[", f);
    for (int k = 0; k < OMNI_TOP; k++) fprintf(f, k ? ",%.9g" : "%.9g", r->weights[k]);
    fprintf(f, "],\"margin\":%.17g}\n", best[OMNI_TOP - 1] - best[OMNI_TOP]);
}

bool clef_gpu_dump_routes(clef_gpu *g, const char *path, char *err, size_t errlen) {
    if (!g || !g->omni || !g->trace || !g->trace_rows || !g->trace_valid) {
        set_err(err, errlen, "no captured Omni routes");
        return false;
    }
    cudaSetDevice(g->device);
    const size_t n = (size_t)g->trace_layers * g->trace_rows;
    omni_route_row *rows = malloc(n * sizeof *rows);
    if (!rows) { set_err(err, errlen, "cannot allocate Omni route dump"); return false; }
    const char *defect = NULL;
    if (cudaMemcpy(rows, g->trace, n * sizeof *rows, cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        defect = "cannot read captured Omni routes";
    }
    for (size_t i = 0; i < n && !defect; i++) defect = route_row_defect(rows + i);
    if (defect) { free(rows); set_err(err, errlen, "%s", defect); return false; }
    FILE *f = fopen(path, "w");
    if (!f) { free(rows); set_err(err, errlen, "cannot open Omni route dump: %s", path); return false; }
    for (size_t i = 0; i < n; i++)
        route_row_print(f, (int)(i / (size_t)g->trace_rows), g->trace_first + (int)(i % (size_t)g->trace_rows), rows + i);
    const bool wrote = !ferror(f);
    const bool closed = fclose(f) == 0;
    free(rows);
    if (!wrote || !closed) { set_err(err, errlen, "cannot write Omni route dump: %s", path); return false; }
    return true;
}

/* ---------------------------------------------------------------- weights */
bool clef_omni_bind_layer(clef_gpu *g, int layer, const void *router, const void *gate_up, const void *down,
                          const float *router_bias, int where, char *err, size_t errlen) {
    if (!g || layer < 0 || layer >= MAX_LAYERS || !router || !gate_up || !down ||
        (where != CLEF_OMNI_HOST && where != CLEF_OMNI_DEVICE)) {
        set_err(err, errlen, "cuda: invalid Omni expert tensor binding");
        return false;
    }
    cudaSetDevice(g->device);
    /* with expert parallelism on, only this rank's contiguous expert range lives here */
    const int world = g->ep.world > 1 ? g->ep.world : 1, EL = OMNI_E / world;
    const size_t per_gu = (size_t)2 * OMNI_F * OMNI_H * 2, per_dn = (size_t)OMNI_H * OMNI_F * 2;
    const size_t nr = (size_t)OMNI_E * OMNI_H * 2, ng = (size_t)EL * per_gu, nd = (size_t)EL * per_dn;
    const size_t first = world > 1 ? (size_t)g->ep.rank * EL : 0;
    omni_layer next;
    memset(&next, 0, sizeof next);
    if (where == CLEF_OMNI_DEVICE) {
        if (((uintptr_t)router | (uintptr_t)gate_up | (uintptr_t)down) & 255) {
            set_err(err, errlen, "cuda: Omni expert tensors must be 256-byte aligned");
            return false;
        }
        next.router = (void *)router; next.gate_up = (void *)gate_up; next.down = (void *)down; next.bias = (float *)router_bias;
    } else {
        next.owned = true;
        next.router = dev_alloc(g, nr); next.gate_up = dev_alloc(g, ng); next.down = dev_alloc(g, nd);
        if (router_bias) next.bias = dev_alloc(g, OMNI_E * 4);
        bool ok = next.router && next.gate_up && next.down && (!router_bias || next.bias);
        if (ok) ok = cudaMemcpyAsync(next.router, router, nr, cudaMemcpyHostToDevice, g->stream) == cudaSuccess &&
                     cudaMemcpyAsync(next.gate_up, (const char *)gate_up + first * per_gu, ng, cudaMemcpyHostToDevice, g->stream) == cudaSuccess &&
                     cudaMemcpyAsync(next.down, (const char *)down + first * per_dn, nd, cudaMemcpyHostToDevice, g->stream) == cudaSuccess &&
                     (!router_bias || cudaMemcpyAsync(next.bias, router_bias, OMNI_E * 4, cudaMemcpyHostToDevice, g->stream) == cudaSuccess) &&
                     cudaStreamSynchronize(g->stream) == cudaSuccess;
        if (!ok) {
            cudaGetLastError();
            free_layer(&next);
            set_err(err, errlen, "cuda: cannot upload Omni expert tensors of layer %d (previous binding kept)", layer);
            return false;
        }
    }
    if (!make_map(g, &next.tm_router, next.router, OMNI_E, OMNI_H, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_128B) ||
        !make_map(g, &next.tm_gate_up, next.gate_up, (uint64_t)EL * 2 * OMNI_F, OMNI_H, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) ||
        !make_map(g, &next.tm_down, next.down, (uint64_t)EL * OMNI_H, OMNI_F, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) ||
        !make_gate_up3(g, &next.tm_gate_up3, next.gate_up, (uint64_t)EL)) {
        free_layer(&next);
        set_err(err, errlen, "cuda: cannot describe Omni expert tensors of layer %d", layer);
        return false;
    }
    next.bound = true;
    cudaStreamSynchronize(g->stream);
    free_layer(&g->layer[layer]);
    g->layer[layer] = next;
    return true;
}

/* ---------------------------------------------------------------- stages */
static bool check_pass(clef_gpu *g, int layer, bool need_weights, char *err, size_t errlen) {
    if (!g || !g->omni) { set_err(err, errlen, "cuda: Omni arena not reserved"); return false; }
    if (need_weights && (layer < 0 || layer >= MAX_LAYERS || !g->layer[layer].bound)) {
        set_err(err, errlen, "cuda: invalid Omni layer dispatch");
        return false;
    }
    cudaSetDevice(g->device);
    return true;
}

/* Stage marks are only recorded here; nothing waits on them inside a pass. */
static void stage_mark(clef_gpu *g, int i) { if (g->profile) cudaEventRecord(g->ev[g->prof_passes % PROF_SLOTS][i], g->stream); }

/* router + exact pass for one chunk; fills arena ids/weights/logits */
static bool run_router(clef_gpu *g, const omni_layer *L, const void *xn, int rows, bool *have_counts) {
    omni_arena *s = g->omni;
    bool fused = false;
    *have_counts = false;
    /* the flagged-row count is cleared by begin and, after each chunk, by the scan kernel: no
     * memset node sits between the kernels of consecutive layers */
    /* the remainders of the exact logits are only read by route capture */
    float *low = g->trace ? s->logits_low : NULL;
    if (low && !launched(g, "capture reset", cudaMemsetAsync(low, 0, (size_t)rows * OMNI_E * 4, g->stream))) return false;
    if (g->router_impl == 0) {
        CUtensorMap tm_x;
        const int nt = omni_router_tile(rows, g->n_sm);
        if (!make_map(g, &tm_x, xn, (uint64_t)rows, OMNI_H, (uint32_t)nt, CU_TENSOR_MAP_L2_PROMOTION_L2_128B)) {
            note_failure(g, "router activation descriptor", cudaErrorInvalidValue);
            return false;
        }
        /* default: the router kernel also counts the experts per sort segment and the exact
         * pass moves the counts of the rows it re-decides, so no histogram kernel is launched */
        fused = g->fused_router != 0;
        if (!launched(g, "router", omni_launch_router_sm100(&tm_x, nt, &L->tm_router, L->bias, rows, g->router_eps, g->router_exact,
                                                            s->logits, s->ids, s->weights, s->flag_rows, s->n_flag, s->status,
                                                            g->debug_stamps ? s->stamps : NULL, fused ? s->sort.segcount : NULL,
                                                            g->stream))) return false;
    } else {
        if (!launched(g, "router (check kernel)", omni_launch_router_simple(xn, L->router, L->bias, rows, s->logits, g->stream))) return false;
        if (!launched(g, "route", omni_launch_select(s->logits, rows, g->router_eps, g->router_exact, s->ids, s->weights,
                                                     s->flag_rows, s->n_flag, s->status, g->stream))) return false;
    }
    if (!launched(g, "router exact pass", omni_launch_recheck(fused ? s->sort.segcount : NULL, xn, L->router, L->bias, s->logits, low, s->flag_rows,
                                                              s->n_flag, rows, g->router_eps, s->ids, s->weights, s->status, g->stream))) return false;
    *have_counts = fused;
    return true;
}

/* permutation + expert products + combine for one chunk, routing taken from ids/weights */
static bool run_experts(clef_gpu *g, const omni_layer *L, const void *xn, const int32_t *ids, const float *weights,
                        float *x, int rows, bool have_counts) {
    omni_arena *s = g->omni;
    const int rows8 = rows * OMNI_TOP;
    if (!launched(g, "assign", omni_launch_assign(ids, rows, s->sort, have_counts, g->stream))) return false;
    /* the tensor-core gate/up kernel fetches its token rows through rowmap itself; the copy
     * into expert order is only made for the check kernels (or when "fused_gather" is 0) */
    const bool fused = g->gemm_impl == 0 && g->fused_gather;
    if (!fused && !launched(g, "gather", omni_launch_gather(xn, s->sort.rowmap, rows8, s->xg, g->stream))) return false;
    stage_mark(g, 2);
    if (g->gemm_impl == 0 && g->expert_kernel > 0) {
        const int ctas = g->expert_kernel;
        if (!launched(g, "gate/up experts", omni_launch_gateup_pair(ctas, &L->tm_gate_up3, s->tm_xg, s->sort, s->h, NULL, NULL, 1, fused ? xn : NULL,
                                                                    fused ? s->sort.rowmap : NULL, NULL, NULL, g->reserve_sms == 0,
                                                                    g->n_sm - g->reserve_sms, g->stream))) return false;
        stage_mark(g, 3);
        if (!launched(g, "down experts", omni_launch_down_pair(ctas, &L->tm_down, s->tm_h, s->sort, s->d, NULL, NULL, g->reserve_sms == 0,
                                                               g->n_sm - g->reserve_sms, g->stream))) return false;
    } else if (g->gemm_impl == 0) {
        /* the down kernel starts on the SMs the first gate/up blocks leave and takes an expert's rows as
         * soon as they are complete: only when this stream's kernels are chained by dependent launch
         * and the gate/up grid invites its successor */
        const int chain = g->expert_chain && g->reserve_sms == 0;
        if (!launched(g, "gate/up experts", omni_launch_gateup_sm100(&L->tm_gate_up, s->tm_xg, s->sort, s->h, NULL, NULL, 1, fused ? xn : NULL,
                                                                     fused ? s->sort.rowmap : NULL, g->reserve_sms == 0, chain,
                                                                     g->n_sm - g->reserve_sms, g->stream))) return false;
        stage_mark(g, 3);
        if (!launched(g, "down experts", omni_launch_down_sm100(&L->tm_down, s->tm_h, s->sort, s->d, NULL, 0, g->reserve_sms == 0, chain,
                                                                g->n_sm - g->reserve_sms, g->stream))) return false;
    } else {
        if (!launched(g, "gate/up experts (check kernel)", omni_launch_gateup_simple(s->xg, L->gate_up, s->sort.offsets, rows8, s->h, g->stream))) return false;
        stage_mark(g, 3);
        if (!launched(g, "down experts (check kernel)", omni_launch_down_simple(s->h, L->down, s->sort.offsets, rows8, s->d, g->stream))) return false;
    }
    stage_mark(g, 4);
    if (g->wait_residual && !launched(g, "residual upload join", cudaStreamWaitEvent(g->stream, g->residual_uploaded, 0))) return false;
    if (!launched(g, "combine", omni_launch_combine(s->d, ids, weights, s->sort.slots, x, rows, g->stream))) return false;
    stage_mark(g, 5);
    return true;
}

/* Expert-parallel variant of run_experts: rows travel to the ranks that own their experts and
 * back by peer stores, inside the two expert kernels (omni_expert.cu, omni_ep_dev.cuh).
 *
 * Default (ep_fused = 1): plan (+ barrier: every rank knows every rank's counts), then the gate/up
 * kernel, whose spare warps send this rank's token rows to the owners group by group while its
 * token producers wait per group of experts until that group's rows have arrived from every
 * rank; then the down kernel, whose epilogue writes every result row piece straight into the
 * buffer of the rank the token came from; one barrier; combine.  No copy kernel runs and the
 * transfers travel under the products.
 *
 * ep_fused = 0 (for comparison, same bits): a copy kernel dispatches all rows and a barrier
 * follows before the gate/up kernel starts; the way back is the same as above. */
static bool run_experts_ep(clef_gpu *g, const omni_layer *L, const void *xn, const int32_t *ids, const float *weights,
                           float *x, int rows, bool have_counts) {
    omni_arena *s = g->omni;
    const int rows8 = rows * OMNI_TOP;
    const omni_ep_peers *pe = &g->ep.peers;
    const int ctas = g->expert_kernel == 1 ? 1 : 2;
    const int n_gemm = g->n_sm - g->reserve_sms;
    if (g->ep_fused && !launched(g, "expert-parallel buckets", omni_launch_ep_buckets(ids, rows, pe->world, g->ep.tok_slot, g->ep.bucket_cnt,
                                                                                       g->ep.bucket_list, g->stream))) return false;
    if (!launched(g, "assign", omni_launch_assign(ids, rows, s->sort, have_counts, g->stream))) return false;
    if (!launched(g, "expert-parallel plan", omni_launch_ep_plan(pe, ++g->ep.epoch, s->sort, g->ep.send_base, g->ep.n_local_rows, g->ep.need,
                                                                 g->ep.bucket_cnt, g->ep.send_cnt, g->ep.recv_base, g->ep.wait_ns, g->stream))) return false;
    if (g->ep_fused) {
        const omni_ep_send send = {g->ep.tok_slot, g->ep.bucket_list, g->ep.send_cnt, g->ep.recv_base, g->ep.send_base,
                                   s->sort.rowmap, s->sort.offsets, xn};
        stage_mark(g, 2);
        /* the token rows arrive once per source token in xg; the kernel gathers each expert's rows from there through grow */
        if (!launched(g, "gate/up experts + dispatch", omni_launch_gateup_pair(ctas, &L->tm_gate_up3, s->tm_xg, s->sort, s->h, pe->flags[pe->rank] + OMNI_EP_READY_WORD,
                                                                               g->ep.need, omni_ep_group_size(pe->world), s->xg, g->ep.grow, pe, &send,
                                                                               g->reserve_sms == 0, n_gemm, g->stream))) return false;
    } else {
        if (!launched(g, "expert-parallel dispatch", omni_launch_ep_dispatch(pe, xn, s->sort.rowmap, s->sort.offsets, g->ep.send_base, rows8, 0, g->n_sm, g->stream))) return false;
        if (!launched(g, "expert-parallel barrier", omni_launch_ep_barrier(pe, ++g->ep.epoch, s->status, g->ep.wait_ns, g->stream))) return false;
        stage_mark(g, 2);
        if (!launched(g, "gate/up experts", omni_launch_gateup_pair(ctas, &L->tm_gate_up3, s->tm_xg, s->sort, s->h, NULL, NULL, 1, NULL, NULL, NULL, NULL,
                                                                    g->reserve_sms == 0, n_gemm, g->stream))) return false;
    }
    stage_mark(g, 3);
    if (!launched(g, "down experts + return", omni_launch_down_pair(ctas, &L->tm_down, s->tm_h, s->sort, s->d, pe, g->ep.rowinfo, g->reserve_sms == 0, n_gemm, g->stream))) return false;
    stage_mark(g, 4);
    if (!launched(g, "expert-parallel barrier", omni_launch_ep_barrier(pe, ++g->ep.epoch, s->status, g->ep.wait_ns, g->stream))) return false;
    if (g->wait_residual && !launched(g, "residual upload join", cudaStreamWaitEvent(g->stream, g->residual_uploaded, 0))) return false;
    if (!launched(g, "combine", omni_launch_combine(g->ep.dret, ids, weights, s->sort.slots, x, rows, g->stream))) return false;
    stage_mark(g, 5);
    return true;
}

static void book_profile(clef_gpu *g) { if (g->profile) g->prof_passes++; }

/* xn == NULL: the rows are normalised here, chunk by chunk, from the residual x */
static bool encode_chunks(clef_gpu *g, int layer, const void *xn, float *x, int T, int n_seq,
                          const int32_t *seq_bounds, char *err, size_t errlen) {
    if (!check_pass(g, layer, true, err, errlen)) return false;
    if (!x || T <= 0 || n_seq < 1 || ((uintptr_t)xn & 15) || ((uintptr_t)x & 15)) {
        set_err(err, errlen, "cuda: invalid Omni layer dispatch");
        return false;
    }
    if (seq_bounds) {
        bool ok = seq_bounds[0] == 0 && seq_bounds[n_seq] == T;
        for (int i = 0; i < n_seq && ok; i++) ok = seq_bounds[i] < seq_bounds[i + 1];
        if (!ok) { set_err(err, errlen, "cuda: invalid Omni sequence bounds"); return false; }
    } else if (n_seq != 1) {
        set_err(err, errlen, "cuda: invalid Omni sequence bounds");
        return false;
    }
    if (g->failed) { set_err(err, errlen, "%s", g->fail_msg); return false; }
    if (g->ep.world > 1 && g->ep.need_sync) {
        set_err(err, errlen, "cuda: an expert-parallel Omni pass failed on this rank; realign the ranks with clef_omni_ep_sync first");
        return false;
    }
    if (g->ep.world > 1 && T > OMNI_CHUNK) {
        set_err(err, errlen, "cuda: expert-parallel Omni passes take at most %d tokens per rank", OMNI_CHUNK);
        return false;
    }
    const omni_layer *L = &g->layer[layer];
    omni_arena *s = g->omni;
    /* Tokens are independent, so the packed batch is processed in arena-sized chunks
     * regardless of record boundaries; a token's arithmetic never depends on its chunk. */
    for (int start = 0; start < T; start += OMNI_CHUNK) {
        const int rows = T - start < OMNI_CHUNK ? T - start : OMNI_CHUNK;
        const char *xn_c = xn ? (const char *)xn + (size_t)start * OMNI_H * 2 : (const char *)g->xnorm;
        stage_mark(g, 0);
        bool have_counts = false;
        bool ok = xn || launched(g, "rmsnorm", omni_launch_rmsnorm(x + (size_t)start * OMNI_H, g->norm_w[layer], g->norm_eps[layer],
                                                                   rows, g->xnorm, g->stream));
        if (ok) ok = run_router(g, L, xn_c, rows, &have_counts);
        if (ok && g->trace && layer < g->trace_layers && start + rows > g->trace_first)
            ok = launched(g, "route capture", omni_launch_trace(s->logits, s->logits_low, s->ids, s->weights, rows, start, g->trace_first,
                                                                g->trace_rows, layer, g->trace, g->stream));
        stage_mark(g, 1);
        if (ok) ok = g->ep.world > 1 ? run_experts_ep(g, L, xn_c, s->ids, s->weights, x + (size_t)start * OMNI_H, rows, have_counts)
                                     : run_experts(g, L, xn_c, s->ids, s->weights, x + (size_t)start * OMNI_H, rows, have_counts);
        if (!ok) {
            if (g->ep.world > 1) g->ep.need_sync = true;     /* this rank launched fewer barriers than its peers */
            set_err(err, errlen, "%s", g->fail_msg);
            return false;
        }
        book_profile(g);
        g->last_T = rows;
    }
    return true;
}

bool clef_omni_encode_moe(clef_gpu *g, int layer, const void *xn, float *x, int T, int n_seq,
                          const int32_t *seq_bounds, char *err, size_t errlen) {
    if (!xn) { set_err(err, errlen, "cuda: invalid Omni layer dispatch"); return false; }
    return encode_chunks(g, layer, xn, x, T, n_seq, seq_bounds, err, errlen);
}

bool clef_omni_bind_norm(clef_gpu *g, int layer, const float *weight, float eps, int where, char *err, size_t errlen) {
    if (!g || layer < 0 || layer >= MAX_LAYERS || !weight || !(eps > 0.f) || !isfinite(eps) ||
        (where != CLEF_OMNI_HOST && where != CLEF_OMNI_DEVICE)) {
        set_err(err, errlen, "cuda: invalid Omni norm binding");
        return false;
    }
    cudaSetDevice(g->device);
    float *w = g->norm_w[layer] ? g->norm_w[layer] : dev_alloc(g, OMNI_H * 4);
    void *xnorm = g->xnorm ? g->xnorm : dev_alloc(g, (size_t)OMNI_CHUNK * OMNI_H * 2);
    bool ok = w && xnorm;
    if (ok) {
        cudaStreamSynchronize(g->stream);      /* a pass in flight may still read the old weights */
        ok = cudaMemcpyAsync(w, weight, OMNI_H * 4, where == CLEF_OMNI_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice,
                             g->stream) == cudaSuccess && cudaStreamSynchronize(g->stream) == cudaSuccess;
    }
    if (!ok) {
        cudaGetLastError();
        if (w && !g->norm_w[layer]) cudaFree(w);
        if (xnorm && !g->xnorm) cudaFree(xnorm);
        set_err(err, errlen, "cuda: cannot upload the Omni norm weights of layer %d (previous binding kept)", layer);
        return false;
    }
    g->norm_w[layer] = w;
    g->norm_eps[layer] = eps;
    g->xnorm = xnorm;
    return true;
}

bool clef_omni_encode_norm_moe(clef_gpu *g, int layer, float *x, int T, int n_seq, const int32_t *seq_bounds,
                               char *err, size_t errlen) {
    if (!g || layer < 0 || layer >= MAX_LAYERS || !g->norm_w[layer]) {
        set_err(err, errlen, "cuda: invalid Omni layer dispatch (no norm weights bound)");
        return false;
    }
    return encode_chunks(g, layer, NULL, x, T, n_seq, seq_bounds, err, errlen);
}

bool clef_omni_forward_host(clef_gpu *g, int layer, const void *xn_host, float *x_host, int T, int n_seq,
                            const int32_t *seq_bounds, char *err, size_t errlen) {
    if (err && errlen) err[0] = 0;
    if (!check_pass(g, layer, true, err, errlen)) return false;
    if (!xn_host || !x_host || T <= 0) { set_err(err, errlen, "cuda: invalid Omni layer dispatch"); return false; }
    if ((size_t)T > g->stage_cap) {
        void *nx = dev_alloc(g, (size_t)T * OMNI_H * 2), *nr = dev_alloc(g, (size_t)T * OMNI_H * 4);
        if (!nx || !nr) {
            if (nx) cudaFree(nx);
            if (nr) cudaFree(nr);
            set_err(err, errlen, "cuda: cannot allocate Omni activation staging (previous buffers kept)");
            return false;
        }
        cudaStreamSynchronize(g->stream);
        if (g->stage_x) cudaFree(g->stage_x);
        if (g->stage_res) cudaFree(g->stage_res);
        g->stage_x = nx; g->stage_res = nr; g->stage_cap = (size_t)T;
    }
    if (!g->copy_stream) {
        bool ok = cudaStreamCreateWithFlags(&g->copy_stream, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&g->out_stream, cudaStreamNonBlocking) == cudaSuccess;
        for (int i = 0; i < HOST_PIECES && ok; i++)
            ok = cudaEventCreateWithFlags(&g->ev_xn[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&g->ev_res[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&g->ev_done[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok) {
            cudaGetLastError();
            set_err(err, errlen, "cuda: cannot create the Omni transfer streams");
            return false;
        }
    }
    if (seq_bounds) {
        bool ok = n_seq >= 1 && seq_bounds[0] == 0 && seq_bounds[n_seq] == T;
        for (int i = 0; i < n_seq && ok; i++) ok = seq_bounds[i] < seq_bounds[i + 1];
        if (!ok) { set_err(err, errlen, "cuda: invalid Omni sequence bounds"); return false; }
    } else if (n_seq != 1) {
        set_err(err, errlen, "cuda: invalid Omni sequence bounds");
        return false;
    }
    /* The link to the host is the slow part (12 KB up and 8 KB down per token), so the batch is
     * cut into pieces of about 1400 tokens: while one piece is in the kernels the next is
     * being uploaded and the previous one downloaded.  Tokens are independent, so the pieces
     * give the same bits as one pass.  Inside a piece the router and the expert products only
     * need xn; the FP32 residual is first touched by the combine and travels beside them.
     * With expert parallelism every rank must issue the same passes: one piece. */
    /* piece size: where a piece's kernels (0.19 ms of weight streaming + 0.06 us per token) take
     * about as long as its upload (0.22 us per token): ~1400 tokens.  What is left exposed at
     * the end of the call is the last piece's kernels and its download, so the last piece gets
     * half the tokens of the others. */
    int n_piece = g->ep.world > 1 || T <= 1536 ? 1 : (T + 1399) / 1400;
    if (g->host_pieces > 0 && g->ep.world <= 1) n_piece = g->host_pieces;
    if (n_piece > HOST_PIECES) n_piece = HOST_PIECES;
    int cut[HOST_PIECES + 1];
    cut[0] = 0;
    {
        const int unit = n_piece > 1 ? ((int)((2L * T) / (2 * n_piece - 1)) + 127) & ~127 : T;
        for (int i = 1; i < n_piece; i++) cut[i] = cut[i - 1] + unit < T ? cut[i - 1] + unit : T;
        cut[n_piece] = T;
        while (n_piece > 1 && cut[n_piece - 1] >= T) n_piece--;      /* tiny batches: fewer pieces */
    }
    clef_omni_begin(g);
    cudaError_t e = cudaSuccess;
    int n_used = 0;
    for (; n_used < n_piece && e == cudaSuccess; n_used++) {
        const size_t rows = (size_t)(cut[n_used + 1] - cut[n_used]), off = (size_t)cut[n_used] * OMNI_H;
        e = cudaMemcpyAsync((char *)g->stage_x + off * 2, (const char *)xn_host + off * 2, rows * OMNI_H * 2, cudaMemcpyHostToDevice, g->copy_stream);
        if (e == cudaSuccess) e = cudaEventRecord(g->ev_xn[n_used], g->copy_stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync((float *)g->stage_res + off, x_host + off, rows * OMNI_H * 4, cudaMemcpyHostToDevice, g->copy_stream);
        if (e == cudaSuccess) e = cudaEventRecord(g->ev_res[n_used], g->copy_stream);
    }
    if (e != cudaSuccess) {
        cudaStreamSynchronize(g->copy_stream);
        set_err(err, errlen, "cuda: cannot upload Omni activations: %s", cudaGetErrorString(e));
        return false;
    }
    bool encoded = true;
    for (int p = 0; p < n_used && encoded; p++) {
        const int start = cut[p], rows = cut[p + 1] - cut[p];
        const size_t off = (size_t)start * OMNI_H;
        e = cudaStreamWaitEvent(g->stream, g->ev_xn[p], 0);
        g->residual_uploaded = g->ev_res[p];
        g->wait_residual = true;
        encoded = e == cudaSuccess && clef_omni_encode_moe(g, layer, (char *)g->stage_x + off * 2, (float *)g->stage_res + off, rows, 1, NULL, err, errlen);
        g->wait_residual = false;
        if (!encoded) break;
        e = cudaEventRecord(g->ev_done[p], g->stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(g->out_stream, g->ev_done[p], 0);
        if (e == cudaSuccess) e = cudaMemcpyAsync(x_host + off, (float *)g->stage_res + off, (size_t)rows * OMNI_H * 4, cudaMemcpyDeviceToHost, g->out_stream);
        if (e != cudaSuccess) { encoded = false; set_err(err, errlen, "cuda: cannot download Omni residual: %s", cudaGetErrorString(e)); }
    }
    if (!encoded) {
        if (e != cudaSuccess && err && !err[0]) set_err(err, errlen, "cuda: Omni host pass failed: %s", cudaGetErrorString(e));
        cudaStreamSynchronize(g->copy_stream);
        cudaStreamSynchronize(g->stream);
        cudaStreamSynchronize(g->out_stream);
        return false;
    }
    const bool done = clef_omni_complete(g, err, errlen);
    if (cudaStreamSynchronize(g->out_stream) != cudaSuccess && done) {
        set_err(err, errlen, "cuda: cannot download Omni residual");
        return false;
    }
    return done;
}

bool clef_omni_stage_router(clef_gpu *g, int layer, const void *xn, int T, double *logits, char *err, size_t errlen) {
    if (!check_pass(g, layer, true, err, errlen)) return false;
    if (!xn || !logits || T <= 0) { set_err(err, errlen, "cuda: invalid Omni router dispatch"); return false; }
    const omni_layer *L = &g->layer[layer];
    if (!launched(g, "router (exact)", omni_launch_router_exact(xn, L->router, L->bias, T, logits, g->stream))) {
        set_err(err, errlen, "%s", g->fail_msg);
        return false;
    }
    return true;
}

bool clef_omni_stage_route(clef_gpu *g, const float *hi, const float *lo, int rows, int32_t *ids, float *weights,
                           char *err, size_t errlen) {
    if (!check_pass(g, 0, false, err, errlen)) return false;
    if (!hi || !ids || !weights || rows <= 0) { set_err(err, errlen, "cuda: invalid Omni route dispatch"); return false; }
    if (!launched(g, "route", omni_launch_route_pairs(hi, lo, rows, ids, weights, g->omni->status, g->stream))) {
        set_err(err, errlen, "%s", g->fail_msg);
        return false;
    }
    return true;
}

bool clef_omni_stage_assign(clef_gpu *g, const int32_t *ids, int rows, int32_t *counts, int32_t *offsets,
                            int32_t *rowmap, int32_t *slots, char *err, size_t errlen) {
    if (!check_pass(g, 0, false, err, errlen)) return false;
    if (!ids || rows <= 0 || rows > OMNI_CHUNK || !counts || !offsets || !rowmap || !slots) {
        set_err(err, errlen, "cuda: invalid Omni assignment dispatch");
        return false;
    }
    omni_sort_state st = g->omni->sort;
    st.counts = counts; st.offsets = offsets; st.rowmap = rowmap; st.slots = slots;
    if (!launched(g, "assign", omni_launch_assign(ids, rows, st, 0, g->stream))) {
        set_err(err, errlen, "%s", g->fail_msg);
        return false;
    }
    return true;
}

bool clef_omni_stage_experts(clef_gpu *g, int layer, const void *xn, const int32_t *ids, const float *weights,
                             float *x, int T, char *err, size_t errlen) {
    if (!check_pass(g, layer, true, err, errlen)) return false;
    if (!xn || !ids || !weights || !x || T <= 0 || T > OMNI_CHUNK ||
        (((uintptr_t)xn | (uintptr_t)ids | (uintptr_t)weights | (uintptr_t)x) & 15)) {      /* vector loads: 16-byte alignment */
        set_err(err, errlen, "cuda: invalid Omni expert dispatch");
        return false;
    }
    stage_mark(g, 0); stage_mark(g, 1);
    if (!run_experts(g, &g->layer[layer], xn, ids, weights, x, T, false)) { set_err(err, errlen, "%s", g->fail_msg); return false; }
    book_profile(g);
    g->last_T = T;
    return true;
}

/* ---------------------------------------------------------------- introspection */
bool clef_omni_read(clef_gpu *g, const char *what, void *dst, size_t bytes, char *err, size_t errlen) {
    if (!check_pass(g, 0, false, err, errlen)) return false;
    omni_arena *s = g->omni;
    const size_t T = (size_t)g->last_T;
    const void *src = NULL;
    size_t have = 0;
    if (!strcmp(what, "ids")) { src = s->ids; have = T * OMNI_TOP * 4; }
    else if (!strcmp(what, "weights")) { src = s->weights; have = T * OMNI_TOP * 4; }
    else if (!strcmp(what, "logits")) { src = s->logits; have = T * OMNI_E * 4; }
    else if (!strcmp(what, "counts")) { src = s->sort.counts; have = OMNI_E * 4; }
    else if (!strcmp(what, "offsets")) { src = s->sort.offsets; have = (OMNI_E + 1) * 4; }
    else if (!strcmp(what, "rowmap")) { src = s->sort.rowmap; have = T * OMNI_TOP * 4; }
    else if (!strcmp(what, "slots")) { src = s->sort.slots; have = T * OMNI_TOP * 4; }
    else if (!strcmp(what, "status")) { src = s->status; have = 4; }
    else if (!strcmp(what, "rechecked")) { src = s->n_flag + 1; have = 4; }
    else if (!strcmp(what, "n_ttiles")) { src = s->sort.n_ttiles; have = 4; }
    else if (!strcmp(what, "xnorm") && g->xnorm) { src = g->xnorm; have = T * OMNI_H * 2; }
    else if (!strcmp(what, "attn_qkv") && g->at.ready) { src = g->at.p; have = (size_t)OMNI_CHUNK * OMNI_QKV * 2; }
    else if (!strcmp(what, "attn_out") && g->at.ready) { src = g->at.a; have = (size_t)OMNI_CHUNK * OMNI_NH * OMNI_HD * 2; }
    else if (!strcmp(what, "router_stamps")) { src = s->stamps; have = (size_t)(OMNI_CHUNK / 32) * 64; }
    if (!src || !dst || bytes > have || !bytes) { set_err(err, errlen, "cuda: unknown or oversized Omni read: %s", what); return false; }
    cudaError_t e = cudaStreamSynchronize(g->stream);
    if (e == cudaSuccess) e = cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { set_err(err, errlen, "cuda: Omni read failed: %s", cudaGetErrorString(e)); return false; }
    return true;
}

bool clef_omni_set_option(clef_gpu *g, const char *name, long value) {
    if (!g || !name) return false;
    if (!strcmp(name, "debug_poison")) g->debug_poison = value != 0;
    else if (!strcmp(name, "router_exact")) g->router_exact = value != 0;
    else if (!strcmp(name, "router_eps")) { if (value <= 0) return false; g->router_eps = (float)((double)value * 1e-9); }
    else if (!strcmp(name, "gemm")) { if (value < 0 || value > 1) return false; g->gemm_impl = (int)value; }
    else if (!strcmp(name, "router")) { if (value < 0 || value > 1) return false; g->router_impl = (int)value; }
    else if (!strcmp(name, "expert_kernel")) { if (value < 0 || value > 2) return false; g->expert_kernel = (int)value; }
    else if (!strcmp(name, "expert_chain")) g->expert_chain = value != 0;
    else if (!strcmp(name, "longest_first")) { if (!g->omni) return false; g->omni->sort.longest_first = value != 0; }
    else if (!strcmp(name, "profile")) { g->profile = value != 0; g->prof_passes = 0; }
    else if (!strcmp(name, "debug_stamps")) g->debug_stamps = value != 0;
    else if (!strcmp(name, "ep_fused")) g->ep_fused = value != 0;
    else if (!strcmp(name, "ep_wait_ms")) { if (value < 0) return false; g->ep.wait_ns = (uint64_t)value * 1000000ull; }
    else if (!strcmp(name, "dependent_launch")) omni_set_dependent_launch(value != 0);
    else if (!strcmp(name, "fused_router")) g->fused_router = value != 0;
    else if (!strcmp(name, "fused_gather")) g->fused_gather = value != 0;
    else if (!strcmp(name, "host_pieces")) { if (value < 0 || value > HOST_PIECES) return false; g->host_pieces = (int)value; }
    else if (!strcmp(name, "reserve_sms")) { if (value < 0 || value >= g->n_sm) return false; g->reserve_sms = (int)value; }
    else if (!strcmp(name, "alloc_fail_at")) { g->alloc_fail_at = value; g->alloc_count = 0; }
    else if (!strcmp(name, "launch_fail_at")) { g->launch_fail_at = value; g->launch_count = 0; }
    else return false;
    return true;
}

bool clef_omni_profile(clef_gpu *g, float ms[6]) {
    if (!g || !g->profile || !ms) return false;
    cudaSetDevice(g->device);
    for (int i = 0; i < 6; i++) ms[i] = 0;
    const long n = g->prof_passes < PROF_SLOTS ? g->prof_passes : PROF_SLOTS;
    g->prof_passes = 0;
    if (n <= 0 || cudaStreamSynchronize(g->stream) != cudaSuccess) { cudaGetLastError(); return n <= 0; }
    for (long p = 0; p < n; p++) {
        float t = 0;
        for (int i = 0; i < 5; i++)
            if (cudaEventElapsedTime(&t, g->ev[p][i], g->ev[p][i + 1]) == cudaSuccess) ms[i] += t / (float)n;
        if (cudaEventElapsedTime(&t, g->ev[p][0], g->ev[p][5]) == cudaSuccess) ms[5] += t / (float)n;
    }
    cudaGetLastError();
    return true;
}

/* ---------------------------------------------------------------- expert parallelism */
static bool ep_alloc(clef_gpu *g, char *err, size_t errlen) {
    if (g->ep.dret) return true;
    void *dret = dev_alloc(g, (size_t)OMNI_ROWS * OMNI_H * 2);
    int32_t *rowinfo = dev_alloc(g, (size_t)OMNI_ROWS * 4);
    int32_t *counts = dev_alloc(g, (size_t)OMNI_EP_MAX * OMNI_EP_COUNT_STRIDE * 4);
    uint32_t *flags = dev_alloc(g, (size_t)OMNI_EP_FLAG_WORDS * 4);
    int32_t *send_base = dev_alloc(g, (size_t)OMNI_E * 4);
    int32_t *n_local = dev_alloc(g, 256);
    int32_t *need = dev_alloc(g, (size_t)OMNI_E * 4);
    uint32_t *sync_result = dev_alloc(g, 256);
    int32_t *tok_slot = dev_alloc(g, (size_t)OMNI_CHUNK * OMNI_EP_MAX * 4);
    int32_t *bucket_cnt = dev_alloc(g, (size_t)OMNI_EP_BUCKETS * 4);
    int32_t *bucket_list = dev_alloc(g, (size_t)OMNI_EP_BUCKETS * OMNI_CHUNK * 4);
    int32_t *send_cnt = dev_alloc(g, (size_t)OMNI_EP_BUCKETS * 4);
    int32_t *recv_base = dev_alloc(g, (size_t)OMNI_EP_BUCKETS * 4);
    int32_t *grow = dev_alloc(g, (size_t)OMNI_ROWS * 4);
    bool ok = dret && rowinfo && counts && flags && send_base && n_local && need && sync_result && tok_slot && bucket_cnt &&
              bucket_list && send_cnt && recv_base && grow;
    if (ok) ok = cudaMemsetAsync(flags, 0, (size_t)OMNI_EP_FLAG_WORDS * 4, g->stream) == cudaSuccess &&
                 cudaMemsetAsync(need, 0, (size_t)OMNI_E * 4, g->stream) == cudaSuccess &&
                 cudaMemsetAsync(counts, 0, (size_t)OMNI_EP_MAX * OMNI_EP_COUNT_STRIDE * 4, g->stream) == cudaSuccess &&
                 cudaMemsetAsync(bucket_cnt, 0, (size_t)OMNI_EP_BUCKETS * 4, g->stream) == cudaSuccess &&
                 cudaMemsetAsync(n_local, 0, 256, g->stream) == cudaSuccess &&
                 cudaStreamSynchronize(g->stream) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        void *all[] = {dret, rowinfo, counts, flags, send_base, n_local, need, sync_result, tok_slot, bucket_cnt, bucket_list, send_cnt,
                       recv_base, grow};
        for (size_t i = 0; i < sizeof all / sizeof all[0]; i++) if (all[i]) cudaFree(all[i]);
        set_err(err, errlen, "cuda: cannot allocate Omni expert-parallel buffers (previous buffers kept)");
        return false;
    }
    g->ep.dret = dret; g->ep.rowinfo = rowinfo; g->ep.counts = counts; g->ep.flags = flags;
    g->ep.send_base = send_base; g->ep.n_local_rows = n_local; g->ep.need = need;
    g->ep.sync_result = sync_result;
    g->ep.tok_slot = tok_slot; g->ep.bucket_cnt = bucket_cnt; g->ep.bucket_list = bucket_list; g->ep.send_cnt = send_cnt;
    g->ep.recv_base = recv_base; g->ep.grow = grow;
    return true;
}

static void ep_local_buffers(clef_gpu *g, void *out[OMNI_EP_BUFFERS]) {
    out[0] = g->omni->xg; out[1] = g->ep.dret; out[2] = g->ep.rowinfo; out[3] = g->ep.counts; out[4] = g->ep.flags; out[5] = g->ep.grow;
}

static void ep_set_peer(omni_ep_peers *pe, int r, void *const buf[OMNI_EP_BUFFERS]) {
    pe->xg[r] = buf[0]; pe->dret[r] = buf[1]; pe->rowinfo[r] = buf[2]; pe->counts[r] = buf[3]; pe->flags[r] = buf[4]; pe->grow[r] = buf[5];
}

bool clef_omni_ep_export(clef_gpu *g, clef_omni_ipc_handle out[CLEF_OMNI_EP_HANDLES], char *err, size_t errlen) {
    if (!g || !g->omni || !out) { set_err(err, errlen, "cuda: Omni arena not reserved"); return false; }
    cudaSetDevice(g->device);
    if (!ep_alloc(g, err, errlen)) return false;
    void *buf[OMNI_EP_BUFFERS];
    ep_local_buffers(g, buf);
    for (int i = 0; i < OMNI_EP_BUFFERS; i++) {
        cudaIpcMemHandle_t h;
        cudaError_t e = cudaIpcGetMemHandle(&h, buf[i]);
        if (e != cudaSuccess) { set_err(err, errlen, "cuda: cannot export Omni exchange buffer %d: %s", i, cudaGetErrorString(e)); return false; }
        memcpy(out[i].reserved, &h, sizeof h);
    }
    return true;
}

static bool ep_check(clef_gpu *g, int rank, int world, char *err, size_t errlen) {
    if (!g || !g->omni) { set_err(err, errlen, "cuda: Omni arena not reserved"); return false; }
    if (world < 2 || world > OMNI_EP_MAX || (OMNI_E % world) || rank < 0 || rank >= world) {
        set_err(err, errlen, "cuda: invalid Omni expert-parallel geometry (rank %d of %d)", rank, world);
        return false;
    }
    if (g->ep.world > 1) { set_err(err, errlen, "cuda: Omni expert parallelism already connected"); return false; }
    for (int l = 0; l < MAX_LAYERS; l++) if (g->layer[l].bound) {
        set_err(err, errlen, "cuda: connect Omni expert parallelism before binding layer weights");
        return false;
    }
    return true;
}

bool clef_omni_ep_connect(clef_gpu *g, int rank, int world, const clef_omni_ipc_handle *all, char *err, size_t errlen) {
    if (!ep_check(g, rank, world, err, errlen)) return false;
    if (!all) { set_err(err, errlen, "cuda: missing Omni exchange handles"); return false; }
    cudaSetDevice(g->device);
    if (!ep_alloc(g, err, errlen)) return false;
    omni_ep_peers pe;
    memset(&pe, 0, sizeof pe);
    pe.rank = rank; pe.world = world;
    memset(g->ep.opened, 0, sizeof g->ep.opened);
    for (int r = 0; r < world; r++) {
        void *buf[OMNI_EP_BUFFERS];
        if (r == rank) ep_local_buffers(g, buf);
        else for (int i = 0; i < OMNI_EP_BUFFERS; i++) {
            cudaIpcMemHandle_t h;
            memcpy(&h, all[r * OMNI_EP_BUFFERS + i].reserved, sizeof h);
            cudaError_t e = cudaIpcOpenMemHandle(&buf[i], h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                cudaGetLastError();
                for (int rr = 0; rr <= r; rr++) for (int ii = 0; ii < OMNI_EP_BUFFERS; ii++)
                    if (g->ep.opened[rr][ii]) { cudaIpcCloseMemHandle(g->ep.opened[rr][ii]); g->ep.opened[rr][ii] = NULL; }
                set_err(err, errlen, "cuda: cannot map rank %d's Omni exchange buffer %d: %s", r, i, cudaGetErrorString(e));
                return false;
            }
            g->ep.opened[r][i] = buf[i];
        }
        ep_set_peer(&pe, r, buf);
    }
    g->ep.peers = pe; g->ep.rank = rank; g->ep.world = world; g->ep.ipc = true; g->ep.epoch = 0; g->ep.sync_count = 0; g->ep.need_sync = false;
    return true;
}

bool clef_omni_ep_connect_local(clef_gpu *g, int rank, int world, clef_gpu *const *peers, char *err, size_t errlen) {
    if (!ep_check(g, rank, world, err, errlen)) return false;
    if (!peers || peers[rank] != g) { set_err(err, errlen, "cuda: invalid Omni peer list"); return false; }
    omni_ep_peers pe;
    memset(&pe, 0, sizeof pe);
    pe.rank = rank; pe.world = world;
    for (int r = 0; r < world; r++) {
        clef_gpu *p = peers[r];
        if (!p || !p->omni) { set_err(err, errlen, "cuda: Omni peer %d has no arena", r); return false; }
        cudaSetDevice(p->device);
        if (!ep_alloc(p, err, errlen)) return false;
        if (p != g) {
            cudaSetDevice(g->device);
            cudaError_t e = cudaDeviceEnablePeerAccess(p->device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
                cudaGetLastError();
                set_err(err, errlen, "cuda: no peer access from device %d to device %d: %s", g->device, p->device, cudaGetErrorString(e));
                return false;
            }
            cudaGetLastError();
        }
        void *buf[OMNI_EP_BUFFERS];
        ep_local_buffers(p, buf);
        ep_set_peer(&pe, r, buf);
    }
    cudaSetDevice(g->device);
    g->ep.peers = pe; g->ep.rank = rank; g->ep.world = world; g->ep.ipc = false; g->ep.epoch = 0; g->ep.sync_count = 0; g->ep.need_sync = false;
    return true;
}

bool clef_omni_ep_sync(clef_gpu *g, int timeout_ms, char *err, size_t errlen) {
    if (!g || !g->omni || g->ep.world < 2) { set_err(err, errlen, "cuda: Omni expert parallelism is not connected"); return false; }
    cudaSetDevice(g->device);
    uint32_t status = 0, agreed[2] = {0, 0};
    const int ms = timeout_ms > 0 ? timeout_ms : 2000;
    /* the attempt publishes sync_count + 1; only success keeps it (omni_ep.cu: ep_sync_kernel) */
    cudaError_t e = cudaStreamSynchronize(g->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(g->omni->status, 0, 4, g->stream);
    if (e == cudaSuccess) e = omni_launch_ep_sync(&g->ep.peers, g->ep.sync_count + 1, g->ep.epoch, g->omni->status, g->ep.sync_result,
                                                  (uint64_t)ms * 1000000ull, g->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(g->stream);
    if (e == cudaSuccess) e = cudaMemcpy(&status, g->omni->status, 4, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && !status) e = cudaMemcpy(agreed, g->ep.sync_result, 8, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { set_err(err, errlen, "cuda: Omni rank barrier failed: %s", cudaGetErrorString(e)); return false; }
    if (status) {
        cudaMemset(g->omni->status, 0, 4);
        set_err(err, errlen, "cuda: not every Omni rank reached the barrier within %d ms", ms);
        return false;
    }
    g->ep.sync_count = agreed[0];
    g->ep.epoch = agreed[1];
    g->ep.need_sync = false;
    g->failed = false;
    return true;
}

void clef_omni_ep_disconnect(clef_gpu *g) {
    if (!g) return;
    cudaSetDevice(g->device);
    cudaStreamSynchronize(g->stream);
    if (g->ep.ipc)
        for (int r = 0; r < OMNI_EP_MAX; r++) for (int i = 0; i < OMNI_EP_BUFFERS; i++)
            if (g->ep.opened[r][i]) { cudaIpcCloseMemHandle(g->ep.opened[r][i]); g->ep.opened[r][i] = NULL; }
    void *all[] = {g->ep.dret, g->ep.rowinfo, g->ep.counts, g->ep.flags, g->ep.send_base, g->ep.n_local_rows, g->ep.need, g->ep.sync_result,
                   g->ep.tok_slot, g->ep.bucket_cnt, g->ep.bucket_list, g->ep.send_cnt, g->ep.recv_base, g->ep.grow};
    for (size_t i = 0; i < sizeof all / sizeof all[0]; i++) if (all[i]) cudaFree(all[i]);
    memset(&g->ep, 0, sizeof g->ep);
    cudaGetLastError();
}

/* ---------------------------------------------------------------- allocation-free entry point */
bool clef_omni_assign_noalloc(const int32_t *ids, int rows, int32_t *counts, int32_t *offsets, int32_t *rowmap,
                              int32_t *slots, uint32_t *status, void *stream, char *err, size_t errlen) {
    int max_rows = 0;
    if (!ids || !counts || !offsets || !rowmap || !slots) {
        set_err(err, errlen, "cuda: invalid Omni assignment dispatch");
        return false;
    }
    cudaError_t e = omni_noalloc_assign(ids, rows, counts, offsets, rowmap, slots, status, (cudaStream_t)stream, &max_rows);
    if (e == cudaSuccess) return true;
    cudaGetLastError();
    if (rows <= 0 || rows > max_rows)
        set_err(err, errlen, "cuda: allocation-free Omni assignment takes 1..%d tokens, got %d", max_rows, rows);
    else
        set_err(err, errlen, "cuda: allocation-free Omni assignment failed: %s", cudaGetErrorString(e));
    return false;
}

/* ---------------------------------------------------------------- attention half */
enum { ATTN_VPITCH = 2 * OMNI_CHUNK, ATTN_MAX_TILES = OMNI_CHUNK / 128 + 4096 };

static void attn_free(clef_gpu *g) {
    void *dev[] = {g->at.p, g->at.q, g->at.k, g->at.vt, g->at.a, g->at.tiles, g->at.vcol, g->at.sched};
    for (size_t i = 0; i < sizeof dev / sizeof dev[0]; i++) if (dev[i]) cudaFree(dev[i]);
    free(g->at.h_tiles); free(g->at.h_vcol); free(g->at.h_bounds);
    memset(&g->at, 0, sizeof g->at);
    for (int l = 0; l < MAX_LAYERS; l++) {
        void *w[] = {g->attn[l].norm_w, g->attn[l].q_norm, g->attn[l].k_norm, g->attn[l].qkv, g->attn[l].out};
        for (size_t i = 0; i < sizeof w / sizeof w[0]; i++) if (w[i]) cudaFree(w[i]);
        memset(&g->attn[l], 0, sizeof g->attn[l]);
    }
}

/* scratch of the attention half, allocated with the first binding: 0.6 GB, independent of T */
static bool attn_reserve(clef_gpu *g, char *err, size_t errlen) {
    if (g->at.ready) return true;
    struct { void **p; size_t bytes; } want[] = {
        {&g->at.p, (size_t)OMNI_CHUNK * OMNI_QKV * 2},
        {&g->at.q, (size_t)OMNI_NH * OMNI_CHUNK * OMNI_HD * 2},
        {&g->at.k, (size_t)OMNI_NKV * OMNI_CHUNK * OMNI_HD * 2},
        {&g->at.vt, (size_t)OMNI_NKV * OMNI_HD * ATTN_VPITCH * 2},
        {&g->at.a, (size_t)OMNI_CHUNK * OMNI_NH * OMNI_HD * 2},
        {(void **)&g->at.tiles, (size_t)ATTN_MAX_TILES * 16},
        {(void **)&g->at.vcol, (size_t)OMNI_CHUNK * 4},
        {(void **)&g->at.sched, 256},
    };
    void *xnorm = g->xnorm ? g->xnorm : dev_alloc(g, (size_t)OMNI_CHUNK * OMNI_H * 2);
    bool ok = xnorm != NULL;
    for (size_t i = 0; i < sizeof want / sizeof want[0] && ok; i++) ok = (*want[i].p = dev_alloc(g, want[i].bytes)) != NULL;
    g->at.h_tiles = malloc((size_t)ATTN_MAX_TILES * 16);
    g->at.h_vcol = malloc((size_t)OMNI_CHUNK * 4);
    g->at.h_bounds = malloc((size_t)(OMNI_CHUNK + 2) * 4);
    ok = ok && g->at.h_tiles && g->at.h_vcol && g->at.h_bounds;
    /* the padding columns of Vt are multiplied by probabilities that are exactly zero: they must stay finite */
    if (ok) ok = cudaMemsetAsync(g->at.vt, 0, (size_t)OMNI_NKV * OMNI_HD * ATTN_VPITCH * 2, g->stream) == cudaSuccess &&
                 cudaMemsetAsync(g->at.k, 0, (size_t)OMNI_NKV * OMNI_CHUNK * OMNI_HD * 2, g->stream) == cudaSuccess &&
                 cudaMemsetAsync(g->at.q, 0, (size_t)OMNI_NH * OMNI_CHUNK * OMNI_HD * 2, g->stream) == cudaSuccess &&
                 cudaStreamSynchronize(g->stream) == cudaSuccess;
    for (int i = 0; i < 4 && ok; i++)
        ok = make_map(g, &g->at.tm_xn[i], xnorm, OMNI_CHUNK, OMNI_H, 32u << i, CU_TENSOR_MAP_L2_PROMOTION_L2_128B) &&
             make_map(g, &g->at.tm_a[i], g->at.a, OMNI_CHUNK, OMNI_NH * OMNI_HD, 32u << i, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (ok) ok = make_map(g, &g->at.tm_q, g->at.q, (uint64_t)OMNI_NH * OMNI_CHUNK, OMNI_HD, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_128B) &&
                 make_map(g, &g->at.tm_k, g->at.k, (uint64_t)OMNI_NKV * OMNI_CHUNK, OMNI_HD, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_128B) &&
                 make_map(g, &g->at.tm_vt, g->at.vt, (uint64_t)OMNI_NKV * OMNI_HD, ATTN_VPITCH, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (!ok) {
        cudaGetLastError();
        if (xnorm && !g->xnorm) cudaFree(xnorm);
        void *dev[] = {g->at.p, g->at.q, g->at.k, g->at.vt, g->at.a, g->at.tiles, g->at.vcol, g->at.sched};
        for (size_t i = 0; i < sizeof dev / sizeof dev[0]; i++) if (dev[i]) cudaFree(dev[i]);
        free(g->at.h_tiles); free(g->at.h_vcol); free(g->at.h_bounds);
        memset(&g->at, 0, sizeof g->at);
        set_err(err, errlen, "cuda: cannot allocate Omni attention scratch (previous buffers kept)");
        return false;
    }
    g->xnorm = xnorm;
    g->at.ready = true;
    g->at.last_T = -1;
    return true;
}

bool clef_omni_bind_attention(clef_gpu *g, int layer, const float *attn_norm, const void *attn_qkv, const void *attn_output,
                              const float *q_norm, const float *k_norm, float eps, float rope_theta, int where, char *err,
                              size_t errlen) {
    if (!g || !g->omni || layer < 0 || layer >= MAX_LAYERS || !attn_norm || !attn_qkv || !attn_output || !q_norm || !k_norm ||
        !(eps > 0.f) || !isfinite(eps) || !(rope_theta > 1.f) || (where != CLEF_OMNI_HOST && where != CLEF_OMNI_DEVICE)) {
        set_err(err, errlen, "cuda: invalid Omni attention binding");
        return false;
    }
    cudaSetDevice(g->device);
    if (!attn_reserve(g, err, errlen)) return false;
    const size_t nq = (size_t)OMNI_QKV * OMNI_H * 2, no = (size_t)OMNI_H * OMNI_NH * OMNI_HD * 2;
    const enum cudaMemcpyKind kind = where == CLEF_OMNI_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice;
    float *nw = dev_alloc(g, OMNI_H * 4), *qn = dev_alloc(g, OMNI_HD * 4), *kn = dev_alloc(g, OMNI_HD * 4);
    void *qkv = dev_alloc(g, nq), *out = dev_alloc(g, no);
    bool ok = nw && qn && kn && qkv && out;
    if (ok) ok = cudaMemcpyAsync(nw, attn_norm, OMNI_H * 4, kind, g->stream) == cudaSuccess &&
                 cudaMemcpyAsync(qn, q_norm, OMNI_HD * 4, kind, g->stream) == cudaSuccess &&
                 cudaMemcpyAsync(kn, k_norm, OMNI_HD * 4, kind, g->stream) == cudaSuccess &&
                 cudaMemcpyAsync(qkv, attn_qkv, nq, kind, g->stream) == cudaSuccess &&
                 cudaMemcpyAsync(out, attn_output, no, kind, g->stream) == cudaSuccess &&
                 cudaStreamSynchronize(g->stream) == cudaSuccess;
    CUtensorMap tm_qkv, tm_out;
    if (ok) ok = make_map(g, &tm_qkv, qkv, OMNI_QKV, OMNI_H, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_256B) &&
                 make_map(g, &tm_out, out, OMNI_H, OMNI_NH * OMNI_HD, 128, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (!ok) {
        cudaGetLastError();
        void *w[] = {nw, qn, kn, qkv, out};
        for (size_t i = 0; i < sizeof w / sizeof w[0]; i++) if (w[i]) cudaFree(w[i]);
        set_err(err, errlen, "cuda: cannot upload Omni attention tensors of layer %d (previous binding kept)", layer);
        return false;
    }
    void *old[] = {g->attn[layer].norm_w, g->attn[layer].q_norm, g->attn[layer].k_norm, g->attn[layer].qkv, g->attn[layer].out};
    for (size_t i = 0; i < sizeof old / sizeof old[0]; i++) if (old[i]) cudaFree(old[i]);
    g->attn[layer].norm_w = nw; g->attn[layer].q_norm = qn; g->attn[layer].k_norm = kn; g->attn[layer].qkv = qkv; g->attn[layer].out = out;
    g->attn[layer].eps = eps; g->attn[layer].theta = (double)rope_theta;
    g->attn[layer].tm_qkv = tm_qkv; g->attn[layer].tm_out = tm_out;
    g->attn[layer].bound = true;
    return true;
}

/* Query tiles (<= 128 rows, cut from each record's start) and the Vt column of every token (a
 * record's columns start at a multiple of 64): rebuilt only when the batch's shape changes. */
static bool attn_plan(clef_gpu *g, int T, int n_seq, const int32_t *seq_bounds, char *err, size_t errlen) {
    const int32_t whole[2] = {0, T};
    const int32_t *b = seq_bounds ? seq_bounds : whole;
    if (g->at.last_T == T && g->at.last_nseq == n_seq && !memcmp(g->at.h_bounds, b, (size_t)(n_seq + 1) * 4)) return true;
    int n_tiles = 0, col = 0;
    for (int r = 0; r < n_seq; r++) {
        const int lo = b[r], hi = b[r + 1];
        if (col + (hi - lo) > ATTN_VPITCH || n_tiles + (hi - lo + 127) / 128 > ATTN_MAX_TILES) {
            set_err(err, errlen, "cuda: too many records in one Omni attention pass (%d)", n_seq);
            return false;
        }
        for (int q0 = lo; q0 < hi; q0 += 128) {
            int32_t *t = g->at.h_tiles + 4 * n_tiles++;
            t[0] = lo; t[1] = q0; t[2] = hi - q0 < 128 ? hi - q0 : 128; t[3] = col;
        }
        for (int t = lo; t < hi; t++) g->at.h_vcol[t] = col + (t - lo);
        col = (col + (hi - lo) + 63) & ~63;
    }
    /* longest first (most key blocks = largest distance from the record's start): the blocks of the
     * grid are dealt in this order, so the short tiles fill the end of the launch.  Insertion sort
     * by distance, descending, stable. */
    for (int i = 1; i < n_tiles; i++) {
        int32_t t[4];
        memcpy(t, g->at.h_tiles + 4 * i, 16);
        const int key = t[1] - t[0];
        int j = i;
        while (j > 0 && g->at.h_tiles[4 * (j - 1) + 1] - g->at.h_tiles[4 * (j - 1)] < key) {
            memcpy(g->at.h_tiles + 4 * j, g->at.h_tiles + 4 * (j - 1), 16);
            j--;
        }
        memcpy(g->at.h_tiles + 4 * j, t, 16);
    }
    if (cudaMemcpyAsync(g->at.tiles, g->at.h_tiles, (size_t)n_tiles * 16, cudaMemcpyHostToDevice, g->stream) != cudaSuccess ||
        cudaMemcpyAsync(g->at.vcol, g->at.h_vcol, (size_t)T * 4, cudaMemcpyHostToDevice, g->stream) != cudaSuccess) {
        cudaGetLastError();
        g->at.last_T = -1;
        set_err(err, errlen, "cuda: cannot upload the Omni attention plan");
        return false;
    }
    memcpy(g->at.h_bounds, b, (size_t)(n_seq + 1) * 4);
    g->at.n_tiles = n_tiles; g->at.last_T = T; g->at.last_nseq = n_seq;
    return true;
}

bool clef_omni_encode_attention(clef_gpu *g, int layer, float *x, const int32_t *pos3, int T, int n_seq,
                                const int32_t *seq_bounds, char *err, size_t errlen) {
    if (!g || !g->omni || layer < 0 || layer >= MAX_LAYERS || !g->attn[layer].bound) {
        set_err(err, errlen, "cuda: invalid Omni layer dispatch (no attention tensors bound)");
        return false;
    }
    if (!x || !pos3 || T <= 0 || T > OMNI_CHUNK || n_seq < 1 || ((uintptr_t)x & 15)) {
        set_err(err, errlen, T > OMNI_CHUNK ? "cuda: an Omni attention pass takes at most 16384 tokens" : "cuda: invalid Omni layer dispatch");
        return false;
    }
    if (seq_bounds) {
        bool ok = seq_bounds[0] == 0 && seq_bounds[n_seq] == T;
        for (int i = 0; i < n_seq && ok; i++) ok = seq_bounds[i] < seq_bounds[i + 1];
        if (!ok) { set_err(err, errlen, "cuda: invalid Omni sequence bounds"); return false; }
    } else if (n_seq != 1) {
        set_err(err, errlen, "cuda: invalid Omni sequence bounds");
        return false;
    }
    cudaSetDevice(g->device);
    if (g->failed) { set_err(err, errlen, "%s", g->fail_msg); return false; }
    if (!attn_plan(g, T, n_seq, seq_bounds, err, errlen)) return false;
    omni_arena *s = g->omni;
    bool ok = launched(g, "attention norm", omni_launch_rmsnorm(x, g->attn[layer].norm_w, g->attn[layer].eps, T, g->xnorm, g->stream)) &&
              launched(g, "projection tiles", omni_launch_dense_tiles(T, s->sort.ttiles, s->sort.n_ttiles, g->at.sched, g->stream)) &&
              launched(g, "q|k|v projection", omni_launch_dense_pair(0, &g->attn[layer].tm_qkv, g->at.tm_xn, s->sort, g->at.sched, g->at.p, NULL,
                                                                       g->n_sm, g->stream)) &&
              launched(g, "attention prep", omni_launch_attn_prep(g->at.p, g->attn[layer].q_norm, g->attn[layer].k_norm, pos3, g->at.vcol, T, OMNI_CHUNK,
                                                                   ATTN_VPITCH, g->attn[layer].eps, g->attn[layer].theta, g->at.q, g->at.k, g->at.vt,
                                                                   s->status, g->stream)) &&
              launched(g, "attention", omni_launch_attention(&g->at.tm_q, &g->at.tm_k, &g->at.tm_vt, g->at.tiles, g->at.n_tiles, OMNI_CHUNK, g->at.a,
                                                             s->status, g->stream)) &&
              launched(g, "output projection", omni_launch_dense_pair(1, &g->attn[layer].tm_out, g->at.tm_a, s->sort, g->at.sched + 1, NULL, x,
                                                                        g->n_sm, g->stream));
    if (!ok) { set_err(err, errlen, "%s", g->fail_msg); return false; }
    return true;
}

/* clef_omni_encode_layer (clef_metal_omni.m:248-331): the attention half, then norm(ffn_norm) and
 * the MoE section, both adding into the same residual stream. */
bool clef_omni_encode_layer(clef_gpu *g, int layer, float *x, const int32_t *pos3, int T, int n_seq, const int32_t *seq_bounds,
                            char *err, size_t errlen) {
    if (!clef_omni_encode_attention(g, layer, x, pos3, T, n_seq, seq_bounds, err, errlen)) return false;
    return clef_omni_encode_norm_moe(g, layer, x, T, n_seq, seq_bounds, err, errlen);
}
