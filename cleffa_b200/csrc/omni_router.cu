// Router of the Clef-Omni MoE block on tcgen05 (sm_100a): logits = x[T][2048] . W_r[128][2048]^T
// with the FP32 accumulator in tensor memory, fused with bias, nonfinite check, top-8 selection,
// renormalised weights, the near-tie flagging that feeds the exact pass
// (reference: metal/clef.metal:2330-2394, omni_router + omni_route) and the per-segment expert
// counts of the counting sort (metal/clef.metal:2396-2410, omni_assign_count).
//
// Orientation: the 128 EXPERTS are the MMA M dimension, a CTA's NT tokens the N dimension.  A
// CTA of 32 tokens costs a quarter of the tensor time and token traffic of one of 128, so a
// 4096-token batch spreads over 128 SMs instead of 32 (the stage is a latency chain -- load,
// multiply, select -- not a bandwidth problem).  Every CTA reads the whole router matrix
// (512 KiB, resident in L2).  The accumulator comes out expert-major (lane = expert, column =
// token); it is transposed through shared memory so that one thread holds one token's 128
// logits for the selection.  NT = 128 serves long batches with the same code.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "omni_internal.h"
#include "omni_pdl.cuh"
#include "omni_ptx.cuh"

namespace {

// Top-9 of 128 per thread without data-dependent branches or predicates: logits become
// order-preserving unsigned keys whose low 7 bits carry (127 - expert id); bitonic networks of
// min/max sort eight groups of 16 and merge them, keeping the best 16 each time.  Equal values
// order by lower id.  The 7 borrowed bits cost a relative 2^-16 in the comparison, which the
// near-tie threshold accounts for; selected values are re-read at full precision afterwards.
__device__ __forceinline__ void ce_desc(uint32_t &x, uint32_t &y) { const uint32_t hi = max(x, y), lo = min(x, y); x = hi; y = lo; }

template <int OFF, int N>
__device__ __forceinline__ void sort16_desc(uint32_t (&k)[N]) {
#pragma unroll
    for (int size = 2; size <= 16; size <<= 1)
#pragma unroll
        for (int stride = size >> 1; stride > 0; stride >>= 1)
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const int l = i ^ stride;
                if (l > i) {
                    if ((i & size) == 0) ce_desc(k[OFF + i], k[OFF + l]);
                    else ce_desc(k[OFF + l], k[OFF + i]);
                }
            }
}

// k[A..A+16) and k[B..B+16) sorted descending -> k[A..A+16) = their best 16, sorted descending
template <int A, int B, int N>
__device__ __forceinline__ void merge_top16(uint32_t (&k)[N]) {
#pragma unroll
    for (int i = 0; i < 16; i++) k[A + i] = max(k[A + i], k[B + 15 - i]);
#pragma unroll
    for (int stride = 8; stride > 0; stride >>= 1)
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int l = i ^ stride;
            if (l > i) ce_desc(k[A + i], k[A + l]);
        }
}

constexpr int RT_THREADS = 256;                         // warp 0 TMA, 1 MMA, 2 TMEM, 3 spare, 4..7 epilogue

template <int NT> struct RtCfg {
    static constexpr int STAGES = NT == 128 ? 4 : 9;               // a latency chain: as many K slabs in flight as fit
    static constexpr int X_BYTES = NT * BK * 2;                     // NT token rows, 64 K each
    static constexpr int STAGE_BYTES = A_TILE_BYTES + X_BYTES;      // + the 128 expert rows
    static constexpr int PITCH = NT + 1;                            // floats per expert row of the transposed logits
    static constexpr int COL_BYTES = OMNI_E * PITCH * 4;
    static constexpr int CAND_BYTES = NT == 32 ? 4 * 16 * 32 * 4 + 2 * 4 * 32 * 4 : 0;   // quarter-wise candidates of the cooperative selection
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + COL_BYTES + CAND_BYTES + 4 * OMNI_E * 4 + 1024 + 256;
};
static_assert(RtCfg<128>::SMEM_BYTES <= 232448 && RtCfg<32>::SMEM_BYTES <= 232448, "shared memory budget");

template <int NT>
__global__ void __launch_bounds__(RT_THREADS, 1)
router_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
              const float *__restrict__ bias, int T, float eps, int exact_all, float *__restrict__ logits,
              int32_t *__restrict__ ids, float *__restrict__ weights, int32_t *__restrict__ flag_rows,
              int32_t *__restrict__ n_flag, uint32_t *__restrict__ status, unsigned long long *__restrict__ dbg,
              int32_t *__restrict__ segcount) {
    using C = RtCfg<NT>;
    constexpr int KSTAGES = OMNI_H / BK, STAGES = C::STAGES, PITCH = C::PITCH;
    // optional per-CTA timestamps (ns): 0 start, 1 loads issued, 2 MMAs issued, 3 accumulator
    // ready, 4 logits stored, 5 selection stored
    auto stamp = [&](int i) { if (dbg) dbg[blockIdx.x * 8 + i] = globaltimer_ns(); };
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    float *const col = reinterpret_cast<float *>(smem_gen + STAGES * C::STAGE_BYTES);          // [128 experts][PITCH]
    uint32_t *const cand = reinterpret_cast<uint32_t *>(smem_gen + STAGES * C::STAGE_BYTES + C::COL_BYTES);   // NT == 32: [4][16][32] keys, then [4][32] max, [4][32] bad
    int *const hist = reinterpret_cast<int *>(smem_gen + STAGES * C::STAGE_BYTES + C::COL_BYTES + C::CAND_BYTES);   // [4][128]
    const uint32_t bar_base = smem_base + STAGES * C::STAGE_BYTES + C::COL_BYTES + C::CAND_BYTES + 4 * OMNI_E * 4;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t tfull_bar = bar_base + 8u * (2 * STAGES);
    uint8_t *misc = smem_gen + STAGES * C::STAGE_BYTES + C::COL_BYTES + C::CAND_BYTES + 4 * OMNI_E * 4 + 8 * (2 * STAGES + 1);
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(misc + 4);
    volatile int *armed = reinterpret_cast<volatile int *>(misc + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * NT;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); armed[s] = -1; }
        mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tm_x);
        prefetch_tmap(&tm_w);
    }
    if (warp == 2) { tmem_alloc(smem_u32((const void *)tmem_slot), NT); tmem_relinquish(); }
    dep_wait();                 // everything above overlaps the tail of the previous kernel
    dep_launch();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0 && lane == 0) {
        PipeState p;
        stamp(0);
        const uint64_t pol_w = l2_policy_evict_last();          // every CTA reads the router matrix
        for (int ks = 0; ks < KSTAGES; ks++) {
            if (!mbar_wait(empty_bar(p.stage), p.phase ^ 1u, abort_flag, status)) break;
            const uint32_t sa = smem_base + p.stage * C::STAGE_BYTES;
            armed[p.stage] = (int)p.phase;
            mbar_expect_tx(full_bar(p.stage), C::STAGE_BYTES);
            tma_load_2d_hint(sa, &tm_w, ks * BK, 0, full_bar(p.stage), pol_w);
            tma_load_2d(sa + A_TILE_BYTES, &tm_x, ks * BK, row0, full_bar(p.stage));      // rows past T read as zero
            p.advance(STAGES);
        }
        stamp(1);
    } else if (warp == 1 && lane == 0) {
        PipeState p;
        const uint32_t idesc = idesc_bf16(128, NT);
        bool ok = true;
        for (int ks = 0; ks < KSTAGES; ks++) {
            ok = mbar_wait(full_bar(p.stage), p.phase, abort_flag, status);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = smem_base + p.stage * C::STAGE_BYTES;
            const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sa + A_TILE_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 16; k++) umma_bf16(tmem_base, da + 2u * k, db + 2u * k, idesc, (ks | k) ? 1u : 0u);
            umma_commit(empty_bar(p.stage));
            p.advance(STAGES);
        }
        umma_commit(tfull_bar);
        stamp(2);
    } else if (warp >= 4) {
        const int q = warp & 3;
        const bool have = mbar_wait(tfull_bar, 0, abort_flag, status);
        if (have) {
            // this warp's 32 experts (TMEM lanes) x NT tokens (columns) -> col[expert][token]
            tc_fence_after();
            if (threadIdx.x == 128) stamp(3);
            const int e = q * 32 + lane;
            const float b = bias ? __ldg(bias + e) : 0.f;
            const uint32_t t0 = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll
            for (int c = 0; c < NT / 32; c++) {
                uint32_t r[32];
                tmem_ld32(t0 + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; j++) col[e * PITCH + c * 32 + j] = bias ? __uint_as_float(r[j]) + b : __uint_as_float(r[j]);
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");            // the four epilogue warps: col is complete
        // Selection.  NT == 128: one thread per token ranks its 128 logits.  NT == 32: the four
        // warps first rank a quarter of the experts each (thread = token), leave their best 16 in
        // shared memory, and warp 0 merges the four lists -- a third of the dependent chain.
        uint32_t key[NT == 32 ? 64 : OMNI_E];
        float max_abs = 0.f;
        bool bad = false;
        if constexpr (NT == 32) {
            if (have) {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const float v = col[(q * 32 + i) * PITCH + lane];
                    bad |= !(fabsf(v) < CUDART_INF_F);
                    max_abs = fmaxf(max_abs, fabsf(v));
                    const uint32_t u = __float_as_uint(v);
                    const uint32_t ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                    key[i] = (ord & ~127u) | (uint32_t)(127 - (q * 32 + i));
                }
                sort16_desc<0>(key); sort16_desc<16>(key);
                merge_top16<0, 16>(key);
#pragma unroll
                for (int i = 0; i < 16; i++) cand[(q * 16 + i) * 32 + lane] = key[i];
                cand[4 * 16 * 32 + q * 32 + lane] = __float_as_uint(max_abs);
                cand[4 * 16 * 32 + 4 * 32 + q * 32 + lane] = bad ? 1u : 0u;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        const bool selecting = have && (NT == 128 || q == 0);
        if (have && (NT == 128 || q != 0)) {
            // logits to HBM, one 512-byte row per token, four coalesced stores per warp and token
            // (with NT == 32 the three warps that do not select share the tokens)
            const int first = NT == 128 ? q : q - 1, step = NT == 128 ? 4 : 3;
            for (int t = first; t < NT; t += step) {
                const long row = row0 + t;
                if (row < T) {
#pragma unroll
                    for (int k = 0; k < 4; k++) logits[row * OMNI_E + lane + 32 * k] = col[(lane + 32 * k) * PITCH + t];
                }
            }
            if (threadIdx.x == 128 + 32) stamp(4);
        }
        const int et = threadIdx.x - 128;
        const long row = row0 + et;
        if (selecting && et < NT && row < T) {
            if constexpr (NT == 32) {
#pragma unroll
                for (int qq = 0; qq < 4; qq++) {
#pragma unroll
                    for (int i = 0; i < 16; i++) key[qq * 16 + i] = cand[(qq * 16 + i) * 32 + lane];
                    max_abs = fmaxf(max_abs, __uint_as_float(cand[4 * 16 * 32 + qq * 32 + lane]));
                    bad |= cand[4 * 16 * 32 + 4 * 32 + qq * 32 + lane] != 0u;
                }
                merge_top16<0, 16>(key); merge_top16<32, 48>(key);
                merge_top16<0, 32>(key);
            } else {
#pragma unroll
                for (int i = 0; i < OMNI_E; i++) {
                    const float v = col[i * PITCH + et];
                    bad |= !(fabsf(v) < CUDART_INF_F);
                    max_abs = fmaxf(max_abs, fabsf(v));
                    const uint32_t u = __float_as_uint(v);
                    const uint32_t ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                    key[i] = (ord & ~127u) | (uint32_t)(127 - i);
                }
            }
            int4 *ip = reinterpret_cast<int4 *>(ids + row * 8);
            float4 *wp = reinterpret_cast<float4 *>(weights + row * 8);
            if (bad) {
                atomicOr(status, OMNI_ST_NONFINITE);     // clef.metal:2362-2367
                ip[0] = make_int4(0, 1, 2, 3); ip[1] = make_int4(4, 5, 6, 7);
                wp[0] = make_float4(0.f, 0.f, 0.f, 0.f); wp[1] = wp[0];
            } else {
                if constexpr (NT == 128) {
                    sort16_desc<0>(key); sort16_desc<16>(key); sort16_desc<32>(key); sort16_desc<48>(key);
                    sort16_desc<64>(key); sort16_desc<80>(key); sort16_desc<96>(key); sort16_desc<112>(key);
                    merge_top16<0, 16>(key); merge_top16<32, 48>(key); merge_top16<64, 80>(key); merge_top16<96, 112>(key);
                    merge_top16<0, 32>(key); merge_top16<64, 96>(key);
                    merge_top16<0, 64>(key);
                }
                float tv[9]; int ti[9];
#pragma unroll
                for (int r = 0; r < 9; r++) { ti[r] = 127 - (int)(key[r] & 127u); tv[r] = col[ti[r] * PITCH + et]; }
                // near-tie threshold: the row's assumed accumulation error (it grows with the
                // row's largest |logit|) plus what the borrowed key bits can hide
                const float thr = 2.f * omni_row_eps(eps, max_abs) + fmaxf(fabsf(tv[0]), fabsf(tv[8])) * 6.1035156e-5f;   // 2^-14
                bool close = exact_all != 0;
#pragma unroll
                for (int k = 0; k < 8; k++) close |= (tv[k] - tv[k + 1]) < thr;
                float p[8], sum = 0.f;
#pragma unroll
                for (int k = 0; k < 8; k++) { p[k] = expf(tv[k] - tv[0]); sum += p[k]; }
                const float inv = 1.f / sum;
                ip[0] = make_int4(ti[0], ti[1], ti[2], ti[3]); ip[1] = make_int4(ti[4], ti[5], ti[6], ti[7]);
                wp[0] = make_float4(p[0] * inv, p[1] * inv, p[2] * inv, p[3] * inv);
                wp[1] = make_float4(p[4] * inv, p[5] * inv, p[6] * inv, p[7] * inv);
                if (close) { const int at = atomicAdd(n_flag, 1); if (at < OMNI_CHUNK) flag_rows[at] = (int32_t)row; }
            }
        }
        if (threadIdx.x == 128) stamp(5);
        if (segcount && q * 32 < NT) {
            // Each selecting warp's 32 tokens are one 256-assignment segment of the counting sort:
            // count their experts here (the exact pass corrects the counts of the rows it changes).
            int *h = hist + q * OMNI_E;
#pragma unroll
            for (int j = 0; j < 4; j++) h[lane + 32 * j] = 0;
            __syncwarp();
            const long row = row0 + q * 32 + lane;
            if (have && row < T) {
                const int4 a = *reinterpret_cast<const int4 *>(ids + row * 8), b = *reinterpret_cast<const int4 *>(ids + row * 8 + 4);
                atomicAdd(h + a.x, 1); atomicAdd(h + a.y, 1); atomicAdd(h + a.z, 1); atomicAdd(h + a.w, 1);
                atomicAdd(h + b.x, 1); atomicAdd(h + b.y, 1); atomicAdd(h + b.z, 1); atomicAdd(h + b.w, 1);
            }
            __syncwarp();
            const int seg = blockIdx.x * (NT / 32) + q;
            if (seg * OMNI_SEG < T * OMNI_TOP) {
#pragma unroll
                for (int j = 0; j < 4; j++) segcount[(long)seg * OMNI_E + lane + 32 * j] = h[lane + 32 * j];
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            const int par = armed[s];
            if (par < 0) continue;
            const uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(full_bar(s), (uint32_t)par) && globaltimer_ns() - t0 < 50000000ull) {}
        }
        // and the MMAs that may still be reading them
        const uint64_t t0 = globaltimer_ns();
        while (!mbar_try_wait(tfull_bar, 0) && globaltimer_ns() - t0 < 50000000ull) {}
    }
    __syncthreads();
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, NT); }
}

}  // namespace

extern "C" {

cudaError_t omni_router_configure(void) {
    cudaError_t e = cudaFuncSetAttribute(router_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, RtCfg<32>::SMEM_BYTES);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(router_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, RtCfg<128>::SMEM_BYTES);
}

// Tokens per CTA for a batch of T tokens: 32 while that gives at most one CTA per SM, else 128.
int omni_router_tile(int T, int n_sm) { return (T + 31) / 32 <= n_sm ? 32 : 128; }

// tm_x: map of the activations whose box is 64 K elements x `nt` rows (nt = omni_router_tile)
cudaError_t omni_launch_router_sm100(const CUtensorMap *tm_x, int nt, const CUtensorMap *tm_w, const float *bias, int T,
                                     float eps, int exact_all, float *logits, int32_t *ids, float *weights,
                                     int32_t *flag_rows, int32_t *n_flag, uint32_t *status, unsigned long long *dbg,
                                     int32_t *segcount, cudaStream_t s) {
    if (nt == 32)
        return omni_launch_chain(router_kernel<32>, dim3((T + 31) / 32), dim3(RT_THREADS), RtCfg<32>::SMEM_BYTES, s, *tm_x, *tm_w, bias, T,
                                 eps, exact_all, logits, ids, weights, flag_rows, n_flag, status, dbg, segcount);
    return omni_launch_chain(router_kernel<128>, dim3((T + 127) / 128), dim3(RT_THREADS), RtCfg<128>::SMEM_BYTES, s, *tm_x, *tm_w, bias, T,
                             eps, exact_all, logits, ids, weights, flag_rows, n_flag, status, dbg, segcount);
}

}  // extern "C"
