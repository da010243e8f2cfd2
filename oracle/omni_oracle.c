/* Plain-C restatement of the serial oracles embedded in the reference's model-free tests.
 * TEST INFRASTRUCTURE ONLY: the product never links or calls this file.
 *
 *   oracle_assign_padded     tests/test_omni_assign.m:44-56 (32-row padded stable bucketing)
 *   oracle_assign_canonical  same bucketing with unpadded offsets (the comparable permutation)
 *   oracle_route             tests/test_omni_moe.m:98-104 (stable descending order on hi+lo,
 *                            ties to the lowest id, weights over the eight selected) with
 *                            the nonfinite fallback of metal/clef.metal:2362-2367
 *   oracle_router_dot        tests/test_omni_router.m:42 (FP64 dot of activations and BF16 weights)
 *   oracle_moe_rows          tests/test_omni_moe.m:104-113 (FP64 expert products and combine
 *                            in selection order, residual added once)
 *   oracle_rmsnorm           metal/clef.metal:190-204 / ref/omni_fp64.py:31-32, in FP64
 *                            (the ffn_norm in front of the block)
 *
 * Build: make -C oracle   (produces oracle/_build/libomni_oracle.so)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

static float bf16_to_float(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }

/* ids[live] -> counts[E], offsets[E+1] (runs padded to `pad`), rowmap[padded] (-1 = padding),
 * slots[live].  `top` assignments per token.  Returns the padded row bound, or -1. */
int oracle_assign_padded(const int32_t *ids, int live, int n_expert, int top, int pad,
                         int32_t *counts, int32_t *offsets, int32_t *rowmap, int32_t *slots) {
    int padded = live + (live < n_expert ? live : n_expert) * (pad - 1);
    int64_t *cursor = calloc((size_t)n_expert, sizeof *cursor);
    if (!cursor) return -1;
    memset(counts, 0, (size_t)n_expert * 4);
    for (int i = 0; i < live; i++) {
        if (ids[i] < 0 || ids[i] >= n_expert) { free(cursor); return -1; }
        counts[ids[i]]++;
    }
    offsets[0] = 0;
    for (int e = 0; e < n_expert; e++) offsets[e + 1] = offsets[e] + ((counts[e] + pad - 1) / pad) * pad;
    if (offsets[n_expert] > padded) { free(cursor); return -1; }
    for (int i = 0; i < padded; i++) rowmap[i] = -1;
    for (int i = 0; i < live; i++) {
        int e = ids[i], row = offsets[e] + (int)cursor[e]++;
        rowmap[row] = i / top;
        slots[i] = row;
    }
    free(cursor);
    return padded;
}

int oracle_assign_canonical(const int32_t *ids, int live, int n_expert, int top,
                            int32_t *counts, int32_t *offsets, int32_t *rowmap, int32_t *slots) {
    int64_t *cursor = calloc((size_t)n_expert, sizeof *cursor);
    if (!cursor) return -1;
    memset(counts, 0, (size_t)n_expert * 4);
    for (int i = 0; i < live; i++) {
        if (ids[i] < 0 || ids[i] >= n_expert) { free(cursor); return -1; }
        counts[ids[i]]++;
    }
    offsets[0] = 0;
    for (int e = 0; e < n_expert; e++) offsets[e + 1] = offsets[e] + counts[e];
    for (int i = 0; i < live; i++) {
        int e = ids[i], row = offsets[e] + (int)cursor[e]++;
        rowmap[row] = i / top;
        slots[i] = row;
    }
    free(cursor);
    return live;
}

/* hi/lo FP32 logit pairs [rows][n_expert] -> ids[rows][top], weights[rows][top] (FP64).
 * Returns the status word: bit 0 set when any row held a nonfinite value. */
uint32_t oracle_route(const float *hi, const float *lo, int rows, int n_expert, int top,
                      int32_t *ids, double *weights) {
    uint32_t status = 0;
    int *order = malloc((size_t)n_expert * sizeof *order);
    double *score = malloc((size_t)n_expert * sizeof *score);
    if (!order || !score) { free(order); free(score); return 0x80000000u; }
    for (int t = 0; t < rows; t++) {
        int bad = 0;
        for (int e = 0; e < n_expert; e++) {
            float h = hi[(size_t)t * n_expert + e], l = lo ? lo[(size_t)t * n_expert + e] : 0.0f;
            if (!isfinite(h) || !isfinite(l)) bad = 1;
            score[e] = (double)h + l;
            order[e] = e;
        }
        if (bad) {
            status |= 1u;
            for (int k = 0; k < top; k++) { ids[t * top + k] = k; weights[t * top + k] = 0.0; }
            continue;
        }
        for (int i = 1; i < n_expert; i++) {            /* stable insertion sort, descending */
            int j = i, e = order[i];
            while (j > 0 && score[order[j - 1]] < score[e]) { order[j] = order[j - 1]; j--; }
            order[j] = e;
        }
        double den = 0;
        for (int k = 0; k < top; k++) den += exp(score[order[k]] - score[order[0]]);
        for (int k = 0; k < top; k++) {
            ids[t * top + k] = order[k];
            weights[t * top + k] = exp(score[order[k]] - score[order[0]]) / den;
        }
    }
    free(order); free(score);
    return status;
}

/* logits[t][e] = sum_k x[t][k] * w[e][k] in FP64; x is FP32, w is BF16 bit patterns. */
void oracle_router_dot(const float *x, const uint16_t *w, int rows, int n_expert, int K, double *logits) {
    for (int t = 0; t < rows; t++) for (int e = 0; e < n_expert; e++) {
        double s = 0;
        for (int k = 0; k < K; k++) s += (double)x[(size_t)t * K + k] * bf16_to_float(w[(size_t)e * K + k]);
        logits[(size_t)t * n_expert + e] = s;
    }
}

/* y[t][i] = x[t][i] * (1 / sqrt(mean_i x[t][i]^2 + eps)) * w[i] */
void oracle_rmsnorm(const double *x, const double *w, double eps, int rows, int Hn, double *y) {
    for (int t = 0; t < rows; t++) {
        const double *xr = x + (size_t)t * Hn;
        double ss = 0;
        for (int i = 0; i < Hn; i++) ss += xr[i] * xr[i];
        const double inv = 1.0 / sqrt(ss / Hn + eps);
        for (int i = 0; i < Hn; i++) y[(size_t)t * Hn + i] = xr[i] * inv * w[i];
    }
}

/* y[t][h] = residual[t][h] + sum_j weight[t][j] * sum_f act_j[f] * down[e_j][h][f],
 * act_j[f] = silu(x.gate[e_j][f]) * (x.up[e_j][f]); gate_up is [E][2F][H], down is [E][H][F]. */
void oracle_moe_rows(const float *x, const float *residual, const int32_t *ids, const double *weights,
                     const uint16_t *gate_up, const uint16_t *down, int rows, int Hn, int Fn, int top,
                     double *y) {
    double *act = malloc((size_t)Fn * sizeof *act);
    if (!act) return;
    for (int t = 0; t < rows; t++) {
        for (int h = 0; h < Hn; h++) y[(size_t)t * Hn + h] = 0;
        for (int j = 0; j < top; j++) {
            int e = ids[t * top + j];
            double wgt = weights[t * top + j];
            for (int f = 0; f < Fn; f++) {
                double g = 0, u = 0;
                const uint16_t *gr = gate_up + ((size_t)e * 2 * Fn + f) * Hn;
                const uint16_t *ur = gate_up + ((size_t)e * 2 * Fn + Fn + f) * Hn;
                for (int h = 0; h < Hn; h++) {
                    g += (double)x[(size_t)t * Hn + h] * bf16_to_float(gr[h]);
                    u += (double)x[(size_t)t * Hn + h] * bf16_to_float(ur[h]);
                }
                act[f] = g / (1 + exp(-g)) * u;
            }
            for (int h = 0; h < Hn; h++) {
                const uint16_t *dr = down + ((size_t)e * Hn + h) * Fn;
                double s = 0;
                for (int f = 0; f < Fn; f++) s += act[f] * bf16_to_float(dr[f]);
                y[(size_t)t * Hn + h] += s * wgt;
            }
        }
        if (residual) for (int h = 0; h < Hn; h++) y[(size_t)t * Hn + h] += residual[(size_t)t * Hn + h];
    }
    free(act);
}
