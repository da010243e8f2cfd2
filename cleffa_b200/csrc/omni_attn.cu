// Attention half of a Clef-Omni decoder layer on sm_100a: the step in front of the MoE block.
//   attn_prep_kernel    per-head RMS norm of q and k, interleaved three-axis rotary, q/k/v laid out
//                       per head (reference: metal/clef.metal:2073-2130, omni_attn_prep)
//   attention_kernel    causal grouped-query attention inside each record of the packed batch,
//                       online softmax (reference: metal/clef.metal:2174-2319, omni_attention)
//   dense_tiles_kernel  tile list that lets the expert-product kernel (omni_expert.cu) run the
//                       q|k|v and the output projection as one "expert" over all token rows
//
// attention_kernel: one CTA per (query head, query tile of <= 128 rows of ONE record).  Both
// products run on tcgen05 with operands in 128-byte-swizzled shared memory: S = Q K^T (128 x 128
// keys, accumulator in tensor memory), softmax by 128 threads (one query row each, FP32, running
// maximum and sum), P written back to shared memory as BF16, O_j = P V_j into a second
// accumulator, which the same threads add into their FP32 registers with the usual rescaling.
// Key blocks start at the record's first token, so a token sees the same blocks whether its
// record is packed with others or runs alone.  V is kept transposed ([d][token]) so that both
// products read K-major operands; each record's columns start at a multiple of 64 tokens
// (`vcol`), which keeps every TMA box 16-byte aligned.  Every wait is bounded.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#include "omni_internal.h"
#include "omni_pdl.cuh"
#include "omni_ptx.cuh"

namespace {

constexpr int HD = OMNI_HD, NH = OMNI_NH, NKV = OMNI_NKV;

// ------------------------------------------------------------------ tile list of a dense projection
__global__ void dense_tiles_kernel(int T, omni_ttile *ttiles, int32_t *n_ttiles, int32_t *counters) {
    const int nt = (T + OMNI_TILE_N - 1) / OMNI_TILE_N;
    const int base = T / nt, extra = T % nt;
    for (int j = threadIdx.x; j < nt; j += blockDim.x)
        ttiles[j] = omni_ttile{0, j * base + min(j, extra), base + (j < extra), 0 | (nt << 16)};
    if (threadIdx.x == 0) { *n_ttiles = nt; counters[0] = 0; counters[1] = 0; }
}

// ------------------------------------------------------------------ q/k norm + rotary + layout
// One block per token, four warps, nine heads each (32 query heads, then the 4 key heads): 128
// values per head, four per lane (elements lane + 32 j).  Pair p of a head is (element p, element
// p + 64); its angle is position[axis] * theta^(-p/64) with axis = p % 3 for p < 60 and the
// temporal axis above (sections 24/20/20 interleaved; clef.metal:2051-2053).  The angle is formed
// and reduced modulo 2 pi in FP64 -- FP32 loses ~pos * 6e-8 rad (clef.metal:2055-2060) -- and its
// cosine and sine, the same for every head of the token, are computed once per warp.
__global__ void __launch_bounds__(128) attn_prep_kernel(const __nv_bfloat16 *__restrict__ qkv, const float *__restrict__ qw,
                                                        const float *__restrict__ kw, const int32_t *__restrict__ pos,
                                                        int head_stride, float eps, double theta,
                                                        __nv_bfloat16 *__restrict__ Q, __nv_bfloat16 *__restrict__ K,
                                                        uint32_t *__restrict__ status) {
    dep_wait();
    dep_launch();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long t = blockIdx.x;
    float cs[2], sn[2];
#pragma unroll
    for (int j = 0; j < 2; j++) {
        const int pair = lane + 32 * j, axis = pair < 60 ? pair % 3 : 0;
        const double angle = (double)__ldg(pos + 3 * t + axis) * exp2(-(double)pair * (1.0 / 64.0) * log2(theta));
        const double turns = rint(angle * 0.15915494309189535);
        const float r = (float)fma(-turns, 6.283185307179586, angle);           // |r| <= pi, accurate to FP32 rounding
        sincosf(r, &sn[j], &cs[j]);
    }
    float wq[4], wk[4];
#pragma unroll
    for (int j = 0; j < 4; j++) { wq[j] = __ldg(qw + lane + 32 * j); wk[j] = __ldg(kw + lane + 32 * j); }
    bool bad = false;
    for (int h = warp; h < NH + NKV; h += 4) {
        const bool query = h < NH;
        const __nv_bfloat16 *src = qkv + t * OMNI_QKV + (long)h * HD;
        float x[4], sum = 0.f;
#pragma unroll
        for (int j = 0; j < 4; j++) { x[j] = __bfloat162float(src[lane + 32 * j]); bad |= !(fabsf(x[j]) < CUDART_INF_F); sum += x[j] * x[j]; }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
        const float inv = rsqrtf(sum / (float)HD + eps);
#pragma unroll
        for (int j = 0; j < 4; j++) x[j] = x[j] * inv * (query ? wq[j] : wk[j]);
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const float lo = x[j], hi = x[j + 2];
            x[j] = lo * cs[j] - hi * sn[j];
            x[j + 2] = hi * cs[j] + lo * sn[j];
        }
        __nv_bfloat16 *dst = query ? Q + ((long)h * head_stride + t) * HD : K + ((long)(h - NH) * head_stride + t) * HD;
#pragma unroll
        for (int j = 0; j < 4; j++) { bad |= !(fabsf(x[j]) < CUDART_INF_F); dst[lane + 32 * j] = __float2bfloat16(x[j]); }
    }
    // reported at completion like the reference's status bit 2 (clef.metal:2120)
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(status, OMNI_ST_ATTN_NONFINITE);
}

// Values, transposed: Vt[kh][d][column of the token].  One block per (64 tokens, key/value head):
// rows read whole (256 bytes per token), written as 64-token runs per head dimension.
__global__ void __launch_bounds__(256) v_transpose_kernel(const __nv_bfloat16 *__restrict__ qkv, const int32_t *__restrict__ vcol,
                                                          int T, int vpitch, __nv_bfloat16 *__restrict__ Vt,
                                                          uint32_t *__restrict__ status) {
    __shared__ unsigned short tile[64][HD + 2];
    __shared__ int col[64];
    dep_wait();
    dep_launch();
    const int t0 = blockIdx.x * 64, kh = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    bool bad = false;
    if (threadIdx.x < 64) col[threadIdx.x] = t0 + threadIdx.x < T ? __ldg(vcol + t0 + threadIdx.x) : -1;
    for (int i = warp; i < 64; i += 8) {
        const long t = t0 + i;
        if (t < T) {
            const uint2 v = *reinterpret_cast<const uint2 *>(qkv + t * OMNI_QKV + (long)(NH + NKV + kh) * HD + lane * 4);
            const unsigned short e[4] = {(unsigned short)(v.x & 0xffff), (unsigned short)(v.x >> 16), (unsigned short)(v.y & 0xffff), (unsigned short)(v.y >> 16)};
#pragma unroll
            for (int k = 0; k < 4; k++) { bad |= (e[k] & 0x7f80) == 0x7f80; tile[i][lane * 4 + k] = e[k]; }
        }
    }
    __syncthreads();
    unsigned short *out = reinterpret_cast<unsigned short *>(Vt) + (long)kh * HD * vpitch;
    for (int d = warp; d < HD; d += 8)
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int i = lane + 32 * k;
            if (col[i] >= 0) out[(long)d * vpitch + col[i]] = tile[i][d];
        }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(status, OMNI_ST_ATTN_NONFINITE);
}

// ------------------------------------------------------------------ attention
struct AttnTile { int32_t rec_start, q0, q_len, vcol0; };          // vcol0: Vt column of the record's first token

constexpr int AT_THREADS = 384;                                    // warp 0 loads, 1 MMA, 2 TMEM, 3 spare, 4..11 softmax (two threads per query row)
constexpr int AT_TILE_BYTES = 128 * 128 * 2;                       // 32 KiB: 128 rows x 128 BF16 as two 64-column halves
constexpr int AT_KV_STAGES = 2;
constexpr int AT_SMEM_BYTES = AT_TILE_BYTES * (2 + 2 * AT_KV_STAGES) + 1024 + 64 + 32 + 1024 + 64;     // Q, P, K and Vt stages; barriers; exchange

__global__ void __launch_bounds__(AT_THREADS, 1)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_vt, const AttnTile *__restrict__ tiles, int T, float scale,
                 __nv_bfloat16 *__restrict__ out, uint32_t *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t q_smem = smem_base, p_smem = smem_base + AT_TILE_BYTES;
    auto k_smem = [&](int s) { return smem_base + AT_TILE_BYTES * (2 + s); };
    auto v_smem = [&](int s) { return smem_base + AT_TILE_BYTES * (2 + AT_KV_STAGES + s); };
    const uint32_t bar_base = smem_base + AT_TILE_BYTES * (2 + 2 * AT_KV_STAGES);
    // barriers: q_full, kv_full[2], kv_empty[2], s_full, p_full, o_full
    const uint32_t q_full = bar_base;
    auto kv_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto kv_empty = [&](int s) { return bar_base + 8u * (3 + s); };
    const uint32_t s_full = bar_base + 8u * 5, p_full = bar_base + 8u * 6, o_full = bar_base + 8u * 7;
    uint8_t *misc = smem_gen + AT_TILE_BYTES * (2 + 2 * AT_KV_STAGES) + 64;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(misc + 4);
    volatile int *armed = reinterpret_cast<volatile int *>(misc + 8);          // [3]: q, kv stage 0, kv stage 1 (parity, -1 none)
    volatile int *quit = reinterpret_cast<volatile int *>(misc + 20);          // a softmax thread's wait ran out: all of them leave together
    float *xch = reinterpret_cast<float *>(misc + 32);                         // [2][128] what the two threads of a row tell each other

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const AttnTile tile = tiles[blockIdx.x];
    const int h = blockIdx.y, kh = h / (NH / NKV);
    const int q_last = tile.q0 + tile.q_len - 1;                                // last query row of the tile
    const int n_blocks = (q_last - tile.rec_start) / 128 + 1;                   // key blocks from the record's start to the diagonal

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < AT_KV_STAGES; s++) { mbar_init(kv_full(s), 1); mbar_init(kv_empty(s), 1); }
        mbar_init(s_full, 1); mbar_init(p_full, 256); mbar_init(o_full, 1);
        *abort_flag = 0;
        *quit = 0;
        armed[0] = armed[1] = armed[2] = -1;
        fence_mbar_init();
        prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_vt);
    }
    if (warp == 2) { tmem_alloc(smem_u32((const void *)tmem_slot), 256); tmem_relinquish(); }
    dep_wait();
    dep_launch();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- loads: Q once, then K / Vt blocks
        armed[0] = 0;
        mbar_expect_tx(q_full, AT_TILE_BYTES);
        tma_load_2d(q_smem, &tm_q, 0, h * T + tile.q0, q_full);                        // d 0..63
        tma_load_2d(q_smem + AT_TILE_BYTES / 2, &tm_q, 64, h * T + tile.q0, q_full);   // d 64..127
        PipeState p;
        for (int j = 0; j < n_blocks; j++) {
            if (!mbar_wait(kv_empty(p.stage), p.phase ^ 1u, abort_flag, status)) break;
            const int key0 = tile.rec_start + j * 128;
            armed[1 + p.stage] = (int)p.phase;
            mbar_expect_tx(kv_full(p.stage), 2 * AT_TILE_BYTES);
            tma_load_2d(k_smem(p.stage), &tm_k, 0, kh * T + key0, kv_full(p.stage));
            tma_load_2d(k_smem(p.stage) + AT_TILE_BYTES / 2, &tm_k, 64, kh * T + key0, kv_full(p.stage));
            tma_load_2d(v_smem(p.stage), &tm_vt, tile.vcol0 + j * 128, kh * HD, kv_full(p.stage));            // keys 0..63 of the block
            tma_load_2d(v_smem(p.stage) + AT_TILE_BYTES / 2, &tm_vt, tile.vcol0 + j * 128 + 64, kh * HD, kv_full(p.stage));
            p.advance(AT_KV_STAGES);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------- MMA issuer
        // S_0, then per block: O_j = P_j V_j as soon as P_j is written (the softmax threads are done
        // with S_j by then), and straight after it S_{j+1}, so that the next scores are ready while
        // the softmax threads still add O_j into their registers.
        const uint32_t idesc = idesc_bf16(128, 128);
        auto scores = [&](int stage) {       // S = Q K^T over the 128 head dimensions: two 64-wide halves, four K=16 steps each
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const uint64_t da = smem_desc_sw128(q_smem + half * (AT_TILE_BYTES / 2));
                const uint64_t db = smem_desc_sw128(k_smem(stage) + half * (AT_TILE_BYTES / 2));
#pragma unroll
                for (int k = 0; k < 4; k++) umma_bf16(tmem_s, da + 2u * k, db + 2u * k, idesc, (half | k) ? 1u : 0u);
            }
            umma_commit(s_full);
        };
        PipeState p, nx;
        bool ok = mbar_wait(q_full, 0, abort_flag, status) && mbar_wait(kv_full(0), 0, abort_flag, status);
        if (ok) { tc_fence_after(); scores(0); nx.advance(AT_KV_STAGES); }
        for (int j = 0; j < n_blocks && ok; j++) {
            ok = mbar_wait(p_full, (uint32_t)j & 1u, abort_flag, status);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const uint64_t da = smem_desc_sw128(p_smem + half * (AT_TILE_BYTES / 2));
                const uint64_t db = smem_desc_sw128(v_smem(p.stage) + half * (AT_TILE_BYTES / 2));
#pragma unroll
                for (int k = 0; k < 4; k++) umma_bf16(tmem_o, da + 2u * k, db + 2u * k, idesc, (half | k) ? 1u : 0u);
            }
            umma_commit(kv_empty(p.stage));                // K and Vt of this block are free once both products are done
            umma_commit(o_full);
            p.advance(AT_KV_STAGES);
            if (j + 1 < n_blocks) {
                ok = mbar_wait(kv_full(nx.stage), nx.phase, abort_flag, status);
                if (!ok) break;
                tc_fence_after();
                scores(nx.stage);
                nx.advance(AT_KV_STAGES);
            }
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------- softmax + accumulation: two threads per query row
        // Thread (row r, half hf) owns keys hf*64.. of every score block and head dimensions hf*64.. of
        // the output.  The two threads of a row sit in different warps and exchange their partial
        // row maxima through shared memory at a named barrier; a thread whose wait ran out marks
        // `quit` and still joins that barrier, after which all of them leave together.
        const int q4 = warp & 3, hf = (warp - 4) >> 2;
        const int r = q4 * 32 + lane;                                             // row inside the tile = TMEM lane
        const int qg = tile.q0 + r;                                               // global token index of the row
        const uint32_t lane_addr = ((uint32_t)(q4 * 32) << 16) + hf * 64;
        float acc[64];
#pragma unroll
        for (int d = 0; d < 64; d++) acc[d] = 0.f;
        float m = -CUDART_INF_F, l = 0.f;
        bool alive = true;
        for (int j = 0; j < n_blocks; j++) {
            if (alive) alive = mbar_wait(s_full, (uint32_t)j & 1u, abort_flag, status);
            const int key0 = tile.rec_start + j * 128 + hf * 64;
            float sc[64], pmax = -CUDART_INF_F;
            if (alive) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t t32[32];
                    tmem_ld32(tmem_s + lane_addr + c * 32, t32);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        sc[c * 32 + i] = key0 + c * 32 + i <= qg ? __uint_as_float(t32[i]) * scale : -CUDART_INF_F;
                        pmax = fmaxf(pmax, sc[c * 32 + i]);
                    }
                }
                xch[hf * 128 + r] = pmax;
            } else {
                *quit = 1;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (*quit) break;
            // every block holds at least one key the row may see (tiles and blocks are both cut from
            // the record's start in steps of 128), so the row maximum is finite
            const float mx = fmaxf(m, fmaxf(pmax, xch[(hf ^ 1) * 128 + r]));
            const float corr = __expf(m - mx);
            float sum = 0.f;
            // P = exp(s - mx) as BF16 into the swizzled K-major layout: this thread's 64 keys are one
            // 128-byte row of its half tile, chunk c8 of 8 keys at c8 ^ (r & 7)
            uint8_t *prow = smem_gen + AT_TILE_BYTES + hf * (AT_TILE_BYTES / 2) + r * 128;
#pragma unroll
            for (int c8 = 0; c8 < 8; c8++) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const __nv_bfloat162 b = __floats2bfloat162_rn(__expf(sc[c8 * 8 + 2 * i] - mx), __expf(sc[c8 * 8 + 2 * i + 1] - mx));
                    // the sum uses the rounded probabilities the second product multiplies with
                    sum += __bfloat162float(b.x) + __bfloat162float(b.y);
                    w[i] = *reinterpret_cast<const uint32_t *>(&b);
                }
                *reinterpret_cast<uint4 *>(prow + ((c8 ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
            l = l * corr + sum;
            m = mx;
            tc_fence_before();
            fence_proxy_async_smem();
            mbar_arrive(p_full);
            alive = mbar_wait(o_full, (uint32_t)j & 1u, abort_flag, status);
            if (alive) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 2; c++) {
                    uint32_t t32[32];
                    tmem_ld32(tmem_o + lane_addr + c * 32, t32);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) acc[c * 32 + i] = acc[c * 32 + i] * corr + __uint_as_float(t32[i]);
                }
                tc_fence_before();
            }
        }
        // the row's denominator is the sum of what its two threads added up (same maximum in both)
        if (!alive) *quit = 1;
        xch[hf * 128 + r] = l;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (!*quit && r < tile.q_len) {
            const float lt = l + xch[(hf ^ 1) * 128 + r];
            const float inv = lt > 0.f ? 1.f / lt : 0.f;
            uint4 *dst = reinterpret_cast<uint4 *>(out + (long)qg * (NH * HD) + h * HD + hf * 64);
#pragma unroll
            for (int ch = 0; ch < 8; ch++) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const __nv_bfloat162 b = __floats2bfloat162_rn(acc[ch * 8 + 2 * i] * inv, acc[ch * 8 + 2 * i + 1] * inv);
                    w[i] = *reinterpret_cast<const uint32_t *>(&b);
                }
                dst[ch] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // a wait ran out: give loads already in flight a bounded chance to land
        for (int s = 0; s < 3; s++) {
            const int par = armed[s];
            if (par < 0) continue;
            const uint32_t bar = s == 0 ? q_full : kv_full(s - 1);
            const uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(bar, (uint32_t)par) && globaltimer_ns() - t0 < 50000000ull) {}
        }
    }
    __syncthreads();
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

}  // namespace

extern "C" {

cudaError_t omni_attn_configure(void) {
    return cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES);
}

cudaError_t omni_launch_dense_tiles(int T, omni_ttile *ttiles, int32_t *n_ttiles, int32_t *counters, cudaStream_t s) {
    dense_tiles_kernel<<<1, 128, 0, s>>>(T, ttiles, n_ttiles, counters);
    return cudaGetLastError();
}

cudaError_t omni_launch_attn_prep(const void *qkv, const float *qw, const float *kw, const int32_t *pos, const int32_t *vcol, int T,
                                  int head_stride, int vpitch, float eps, double theta, void *Q, void *K, void *Vt, uint32_t *status,
                                  cudaStream_t s) {
    cudaError_t e = omni_launch_chain(attn_prep_kernel, dim3(T), dim3(128), 0, s, (const __nv_bfloat16 *)qkv, qw, kw, pos, head_stride, eps,
                                      theta, (__nv_bfloat16 *)Q, (__nv_bfloat16 *)K, status);
    if (e != cudaSuccess) return e;
    return omni_launch_chain(v_transpose_kernel, dim3((T + 63) / 64, OMNI_NKV), dim3(256), 0, s, (const __nv_bfloat16 *)qkv, vcol, T, vpitch,
                             (__nv_bfloat16 *)Vt, status);
}

// tiles: [n_tiles] of {record start, first query row, rows (<= 128), Vt column of the record start}
cudaError_t omni_launch_attention(const CUtensorMap *tm_q, const CUtensorMap *tm_k, const CUtensorMap *tm_vt, const void *tiles,
                                  int n_tiles, int T, void *out, uint32_t *status, cudaStream_t s) {
    return omni_launch_chain(attention_kernel, dim3(n_tiles, OMNI_NH), dim3(AT_THREADS), AT_SMEM_BYTES, s, *tm_q, *tm_k, *tm_vt,
                             (const AttnTile *)tiles, T, 1.0f / sqrtf((float)OMNI_HD), (__nv_bfloat16 *)out, status);
}

}  // extern "C"
