/* The binding a maintainer of the reference engine adds to drive the CUDA Omni MoE backend:
 * the same text as the stub in the integration guide.  tests/test_abi.py compiles it against the
 * reference's own clef_engine.h (clef_config, clef_layer_w, gguf_tensor) and links it with the
 * library, so the boundary is checked against the reference's real types. */
#include "clef_engine.h"        /* clef_config, clef_layer_w, gguf_tensor: the reference's header */
#include "clef_cuda_omni.h"     /* included after it: enables the clef_config adapter */

static clef_gpu *G;

bool cuda_backend_open(const clef_engine *e, char *err, size_t errlen) {
    if (!clef_cuda_omni_open(&G, 0, NULL, err, errlen)) return false;
    /* clef_metal.m:1148 calls clef_omni_reserve(g, &e->cfg, T, ...): same arguments here */
    if (!clef_omni_reserve_config(G, &e->cfg, 1, err, errlen)) return false;
    for (int l = 0; l < e->cfg.n_layer; l++) {
        const clef_layer_w *w = &e->w.layer[l];               /* clef_engine.h:35-40 */
        /* gguf_tensor.data points into the mmap'd file (clef_gguf.h:31-39) */
        if (!clef_omni_bind_layer(G, l, w->ffn_router->data, w->ffn_gate_up_exps->data, w->ffn_down_exps->data,
                                  NULL, CLEF_OMNI_HOST, err, errlen))
            return false;
        if (!clef_omni_bind_norm(G, l, (const float *)w->ffn_norm->data, e->cfg.eps, CLEF_OMNI_HOST, err, errlen))
            return false;
        if (!clef_omni_bind_attention(G, l, (const float *)w->attn_norm->data, w->attn_qkv->data, w->attn_output->data,
                                      (const float *)w->attn_q_norm->data, (const float *)w->attn_k_norm->data, e->cfg.eps,
                                      e->cfg.rope_theta, CLEF_OMNI_HOST, err, errlen))
            return false;
    }
    return clef_omni_trace_reserve(G, 1, e->cfg.n_layer, e->route_rows, e->capture_routes, err, errlen);
}

/* one pass over a packed batch: d_x is the FP32 residual stream on the device, [T][H]; d_pos3 the
 * tokens' three rotary positions, [T][3] (clef_record_positions), also on the device */
bool cuda_backend_layers(const clef_engine *e, float *d_x, const int32_t *d_pos3, int T, int n_seq, const int32_t *seq_bounds,
                         char *err, size_t errlen) {
    clef_omni_begin(G);                                        /* once per pass (clef_metal.m:1150) */
    for (int l = 0; l < e->cfg.n_layer; l++)                   /* clef_metal_omni.m:248; or its two halves, */
        if (!clef_omni_encode_layer(G, l, d_x, d_pos3, T, n_seq, seq_bounds, err, errlen)) return false;   /* clef_omni_encode_attention + clef_omni_encode_norm_moe */
    return clef_omni_complete(G, err, errlen);                 /* clef_metal.m:1597 */
}

bool cuda_backend_dump_routes(const char *path, char *err, size_t errlen) {
    return clef_gpu_dump_routes(G, path, err, errlen);         /* clef.c:570 */
}

void cuda_backend_close(void) {
    clef_omni_keepalive(G);
    clef_cuda_omni_close(G);
    G = NULL;
}
