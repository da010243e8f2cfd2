// Device helpers shared by the routing kernels: warp-level top-k in the reference's order,
// the selection write-out, and exact logits (FP64 sums of exact BF16 products) with the
// re-evaluation of one near-tied router row by a group of four warps.
//
// Reference behaviour (paths inside the reference project):
//   selection order / weights   metal/clef.metal:2347-2394  (omni_route)
//   exact logits                metal/clef.metal:2330-2345  (omni_router, compensated sum)
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "omni_internal.h"

namespace {

constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ float bf16_bits_to_float(uint32_t b16) { return __uint_as_float(b16 << 16); }

// ------------------------------------------------------------------ warp-level top-k
// Order: larger value first, equal values -> lower expert id first (clef.metal:2376-2382).
struct Best { double v; int id; };

__device__ __forceinline__ bool better(double v, int id, double ov, int oid) {
    return v > ov || (v == ov && id < oid);
}

__device__ __forceinline__ Best warp_argmax(double v, int id) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const double ov = __shfl_xor_sync(FULL, v, s);
        const int oid = __shfl_xor_sync(FULL, id, s);
        if (better(ov, oid, v, id)) { v = ov; id = oid; }
    }
    return Best{v, id};
}

// Each lane owns experts lane, lane+32, lane+64, lane+96.  Extracts the `n` best (n <= 9)
// in order into top_v/top_id (identical on every lane).  Taken entries become -inf.
template <int N>
__device__ __forceinline__ void warp_topn(double (&val)[4], int lane, double (&top_v)[N], int (&top_id)[N]) {
#pragma unroll
    for (int r = 0; r < N; r++) {
        double bv = val[0]; int bid = lane;
#pragma unroll
        for (int j = 1; j < 4; j++) if (better(val[j], lane + 32 * j, bv, bid)) { bv = val[j]; bid = lane + 32 * j; }
        const Best b = warp_argmax(bv, bid);
        top_v[r] = b.v; top_id[r] = b.id;
#pragma unroll
        for (int j = 0; j < 4; j++) if (lane + 32 * j == b.id) val[j] = -CUDART_INF;
    }
}

// Lanes 0..7 hold the selected logits; weights are softmax over the selected eight, which
// equals softmax over all experts renormalised by the selected sum (clef.metal:2393).
__device__ __forceinline__ void write_selection(const double (&top_v)[9], const int (&top_id)[9], int lane,
                                                int32_t *ids, float *weights, long row) {
    double p = 0.0;
#pragma unroll
    for (int k = 0; k < 8; k++) if (lane == k) p = exp(top_v[k] - top_v[0]);
    double sum = p;
#pragma unroll
    for (int s = 4; s > 0; s >>= 1) sum += __shfl_xor_sync(FULL, sum, s);
    if (lane < 8) {
        int id = 0;
#pragma unroll
        for (int k = 0; k < 8; k++) if (lane == k) id = top_id[k];
        ids[row * 8 + lane] = id;
        weights[row * 8 + lane] = (float)(p / sum);
    }
}

__device__ __forceinline__ void write_fallback(int lane, int32_t *ids, float *weights, long row, uint32_t *status) {
    // clef.metal:2362-2367: report once, keep the pass well-defined.
    if (lane == 0) atomicOr(status, OMNI_ST_NONFINITE);
    if (lane < 8) { ids[row * 8 + lane] = lane; weights[row * 8 + lane] = 0.0f; }
}

// ------------------------------------------------------------------ exact dot (FP64 sum of exact products)
// A lane owns K elements lane*8 + 256*i .. +7 (i < 8): one 16-byte load per step.
struct XRow { uint4 q[8]; };

__device__ __forceinline__ XRow load_xrow(const __nv_bfloat16 *xn, long row, int lane) {
    XRow r;
    const uint4 *p = reinterpret_cast<const uint4 *>(xn + row * OMNI_H);
#pragma unroll
    for (int i = 0; i < 8; i++) r.q[i] = __ldg(p + lane + 32 * i);
    return r;
}

// bf16*bf16 is exact in FP32 (8+8 significand bits); the FP64 sum of 2048 such terms is
// accurate to ~1e-13, far inside the 1e-9 bound of tests/test_omni_router.m:44.
__device__ __forceinline__ double exact_dot(const XRow &x, const __nv_bfloat16 *wrow, int lane) {
    const uint4 *p = reinterpret_cast<const uint4 *>(wrow);
    uint4 w[8];
#pragma unroll
    for (int i = 0; i < 8; i++) w[i] = __ldg(p + lane + 32 * i);
    double acc[4] = {0.0, 0.0, 0.0, 0.0};      // four chains: the FP64 adds overlap instead of serialising
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t xu[4] = {x.q[i].x, x.q[i].y, x.q[i].z, x.q[i].w};
        const uint32_t wu[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            acc[j] += (double)(bf16_bits_to_float(xu[j] & 0xffffu) * bf16_bits_to_float(wu[j] & 0xffffu));
            acc[j] += (double)(bf16_bits_to_float(xu[j] >> 16) * bf16_bits_to_float(wu[j] >> 16));
        }
    }
    double sum = (acc[0] + acc[1]) + (acc[2] + acc[3]);
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(FULL, sum, s);
    return sum;
}

// Re-evaluates one flagged row with four warps (128 threads): exact logits for every expert
// that can still reach the top eight (approximate logit within twice the row's error bound of
// the approximate 8th) and for the approximate 9th, spread over the warps, then the final order
// by warp 0.  `sync` is a barrier over exactly these 128 threads; `exact_s` is their scratch of
// 128 doubles.  With `segcount` given (expert counts per 256-assignment segment, taken from the
// ids being replaced), the counts follow the ids that change.
//
// What the pass learns is written back: every logit it evaluated is replaced by its exact value
// as a float pair (hi into `logits`, the remainder into `low` when given), so that a capture of
// the row shows logits that agree with the ids chosen from them (clef_metal_omni.m:118-130
// prints hi+lo).  And the assumed error bound is checked on the way: an approximate logit
// further than the bound from its exact value raises OMNI_ST_ROUTER_EPS.
template <typename Sync>
__device__ __forceinline__ void recheck_row(const __nv_bfloat16 *__restrict__ xn, const __nv_bfloat16 *__restrict__ w,
                                            const float *__restrict__ bias, float *__restrict__ logits,
                                            float *__restrict__ low, long row, float eps, int32_t *__restrict__ ids,
                                            float *__restrict__ weights, int32_t *__restrict__ segcount,
                                            uint32_t *__restrict__ status, double *exact_s, int lane, int warp, Sync sync) {
    exact_s[warp * 32 + lane] = -CUDART_INF;
    double val[4], approx[4];
    float max_abs = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float f = logits[row * OMNI_E + lane + 32 * j];
        approx[j] = val[j] = (double)f;
        max_abs = fmaxf(max_abs, fabsf(f));
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) max_abs = fmaxf(max_abs, __shfl_xor_sync(FULL, max_abs, s));
    const double bound = (double)omni_row_eps(eps, max_abs);
    const XRow x = load_xrow(xn, row, lane);              // in flight while the threshold is found
    double top_v[9]; int top_id[9];
    warp_topn<9>(val, lane, top_v, top_id);               // every warp finds the same threshold
    const double floor_v = fmin(top_v[7] - 2.0 * bound, top_v[8]);
    sync();
    int c = 0;
    bool off = false;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        unsigned m = __ballot_sync(FULL, approx[j] >= floor_v);
        while (m) {
            const int src = __ffs(m) - 1;
            m &= m - 1;
            const double a = __shfl_sync(FULL, approx[j], src);
            if ((c++ & 3) != warp) continue;              // candidates round-robin over the warps
            const int e = src + 32 * j;
            double v = exact_dot(x, w + (long)e * OMNI_H, lane);
            if (bias) v += (double)bias[e];
            off |= fabs(v - a) > bound;
            if (lane == 0) {
                exact_s[e] = v;
                const float hi = (float)v;
                logits[row * OMNI_E + e] = hi;
                if (low) low[row * OMNI_E + e] = (float)(v - (double)hi);
            }
        }
    }
    if (off && lane == 0) atomicOr(status, OMNI_ST_ROUTER_EPS);
    sync();
    if (warp == 0) {
        double exact[4];
#pragma unroll
        for (int j = 0; j < 4; j++) exact[j] = exact_s[lane + 32 * j];
        double fin_v[9]; int fin_id[9];
        warp_topn<9>(exact, lane, fin_v, fin_id);         // the 9th is unused here
        const int old_id = lane < 8 ? ids[row * 8 + lane] : 0;
        write_selection(fin_v, fin_id, lane, ids, weights, row);
        if (segcount && lane < 8) {
            const int new_id = ids[row * 8 + lane];       // this lane's own store
            if (new_id != old_id) {                       // a row's eight assignments share one segment
                int32_t *c = segcount + (row * OMNI_TOP / OMNI_SEG) * OMNI_E;
                atomicSub(c + old_id, 1);
                atomicAdd(c + new_id, 1);
            }
        }
    }
    sync();
}

}  // namespace
