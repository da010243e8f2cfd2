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
// One CTA per (query head, tile of <= 128 query rows of one record).  Key blocks of 128 run from the
// record's start to the tile's diagonal.  Per block j:
//   S_j = Q K_j^T        tcgen05, FP32 in TMEM, two score buffers so that S_{j+1} is formed while
//                        the softmax threads work on S_j
//   P_j = exp2(c S_j - m)  256 threads, two per query row (64 keys each), BF16 into a swizzled
//                        shared-memory tile
//   O  += P_j V_j        tcgen05, accumulated in TMEM over all blocks
// m is the row's reference maximum.  It follows the running maximum lazily: only when a block's
// maximum exceeds it by more than 2^8 are O and the running sum rescaled (by the softmax threads,
// in TMEM, between two value products); otherwise P simply holds values up to 256.  The result is
// the same softmax; the accumulator never leaves TMEM until the tile is done.
struct AttnTile { int32_t rec_start, q0, q_len, vcol0; };          // vcol0: Vt column of the record's first token

constexpr int AT_THREADS = 384;                                    // warp 0 loads, 1 MMA, 2 TMEM, 3 spare, 4..11 softmax (two threads per query row)
constexpr int AT_TILE_BYTES = 128 * 128 * 2;                       // 32 KiB: 128 rows x 128 BF16 as two 64-column halves
constexpr int AT_KV_STAGES = 2;
constexpr int AT_TMEM_COLS = 512;                                  // S0, S1, O of 128 columns each
constexpr int AT_N_BARS = 14;
constexpr int AT_XCH_BYTES = 2 * 2 * 128 * 4;                      // [block parity][row half][row]
constexpr int AT_SMEM_BYTES = AT_TILE_BYTES * (2 + 2 * AT_KV_STAGES) + 1024 + AT_N_BARS * 8 + 16 + 64 + AT_XCH_BYTES;
#ifndef AT_DBG_KSTEPS
#define AT_DBG_KSTEPS 4
#endif
constexpr float AT_LAZY = 8.f;                                     // log2 of how far a block may exceed the reference maximum

__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(addr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
        : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {          // 2^x, -inf -> 0; relative error ~2^-22, far below BF16's
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// two FP32 lanes per instruction: (a.x * b.x + c.x, a.y * b.y + c.y) and (a.x + b.x, a.y + b.y)
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)),
        "l"(*reinterpret_cast<uint64_t *>(&c)));
    return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(*reinterpret_cast<uint64_t *>(&b)));
    return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

#ifdef AT_DBG_CLOCK
__device__ unsigned long long at_dbg[16];
#define AT_TICK(k) { const long long now_ = clock64(); tk[k] += now_ - tprev; tprev = now_; }
#else
#define AT_TICK(k)
#endif
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
    // barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full, pv_done
    const uint32_t q_full = bar_base;
    auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bar_base + 8u * (3 + s); };
    auto v_full = [&](int s) { return bar_base + 8u * (5 + s); };
    auto v_empty = [&](int s) { return bar_base + 8u * (7 + s); };
    auto s_full = [&](int b) { return bar_base + 8u * (9 + b); };
    const uint32_t p_full = bar_base + 8u * 11, pv_done = bar_base + 8u * 12;
    uint8_t *misc = smem_gen + AT_TILE_BYTES * (2 + 2 * AT_KV_STAGES) + AT_N_BARS * 8;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(misc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(misc + 4);
    volatile int *quit = reinterpret_cast<volatile int *>(misc + 8);           // a softmax thread's wait ran out: all of them leave together
    volatile int *armed = reinterpret_cast<volatile int *>(misc + 16);         // [5]: q, k stages, v stages (parity of the load in flight, -1 none)
    float *xch = reinterpret_cast<float *>(misc + 16 + 64);                    // what the two threads of a row tell each other

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const AttnTile tile = tiles[blockIdx.x];
    const int h = blockIdx.y, kh = h / (NH / NKV);
    const int q_last = tile.q0 + tile.q_len - 1;                                // last query row of the tile
    const int n_blocks = (q_last - tile.rec_start) / 128 + 1;                   // key blocks from the record's start to the diagonal

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < AT_KV_STAGES; s++) {
            mbar_init(k_full(s), 1); mbar_init(k_empty(s), 1); mbar_init(v_full(s), 1); mbar_init(v_empty(s), 1);
            mbar_init(s_full(s), 1);
        }
        mbar_init(p_full, 256); mbar_init(pv_done, 1);
        *abort_flag = 0;
        *quit = 0;
        for (int i = 0; i < 5; i++) armed[i] = -1;
        fence_mbar_init();
        prefetch_tmap(&tm_q); prefetch_tmap(&tm_k); prefetch_tmap(&tm_vt);
    }
    if (warp == 2) { tmem_alloc(smem_u32((const void *)tmem_slot), AT_TMEM_COLS); tmem_relinquish(); }
    dep_wait();
    dep_launch();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 256;

    if (warp == 0 && lane == 0) {
        // ---------------------------------------------------------- loads: Q once, then K one block ahead of Vt
        armed[0] = 0;
        mbar_expect_tx(q_full, AT_TILE_BYTES);
        tma_load_2d(q_smem, &tm_q, 0, h * T + tile.q0, q_full);                        // d 0..63
        tma_load_2d(q_smem + AT_TILE_BYTES / 2, &tm_q, 64, h * T + tile.q0, q_full);   // d 64..127
        PipeState pk, pv;
        auto load_k = [&](int j) {
            if (!mbar_wait(k_empty(pk.stage), pk.phase ^ 1u, abort_flag, status)) return false;
            const int key0 = tile.rec_start + j * 128;
            armed[1 + pk.stage] = (int)pk.phase;
            mbar_expect_tx(k_full(pk.stage), AT_TILE_BYTES);
            tma_load_2d(k_smem(pk.stage), &tm_k, 0, kh * T + key0, k_full(pk.stage));
            tma_load_2d(k_smem(pk.stage) + AT_TILE_BYTES / 2, &tm_k, 64, kh * T + key0, k_full(pk.stage));
            pk.advance(AT_KV_STAGES);
            return true;
        };
        bool ok = load_k(0);
        for (int j = 0; j < n_blocks && ok; j++) {
            if (j + 1 < n_blocks) ok = load_k(j + 1);
            if (!ok || !mbar_wait(v_empty(pv.stage), pv.phase ^ 1u, abort_flag, status)) break;
            armed[3 + pv.stage] = (int)pv.phase;
            mbar_expect_tx(v_full(pv.stage), AT_TILE_BYTES);
            tma_load_2d(v_smem(pv.stage), &tm_vt, tile.vcol0 + j * 128, kh * HD, v_full(pv.stage));            // keys 0..63 of the block
            tma_load_2d(v_smem(pv.stage) + AT_TILE_BYTES / 2, &tm_vt, tile.vcol0 + j * 128 + 64, kh * HD, v_full(pv.stage));
            pv.advance(AT_KV_STAGES);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------------------------------------------------- MMA issuer
        // S_{j+1} goes to the tensor pipe before the wait for P_j, so that it is there when the softmax
        // threads come back; O += P_j V_j follows as soon as P_j is written.
        const uint32_t idesc = idesc_bf16(128, 128);
        PipeState pk, pv;
        auto scores = [&](int j) {       // S = Q K^T over the 128 head dimensions: two 64-wide halves, four K=16 steps each
            if (!mbar_wait(k_full(pk.stage), pk.phase, abort_flag, status)) return false;
            tc_fence_after();
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const uint64_t da = smem_desc_sw128(q_smem + half * (AT_TILE_BYTES / 2));
                const uint64_t db = smem_desc_sw128(k_smem(pk.stage) + half * (AT_TILE_BYTES / 2));
#pragma unroll
                for (int k = 0; k < AT_DBG_KSTEPS; k++) umma_bf16(tmem_base + (j & 1) * 128, da + 2u * k, db + 2u * k, idesc, (half | k) ? 1u : 0u);
            }
            umma_commit(k_empty(pk.stage));
            umma_commit(s_full(j & 1));
            pk.advance(AT_KV_STAGES);
            return true;
        };
        bool ok = mbar_wait(q_full, 0, abort_flag, status) && scores(0);
        for (int j = 0; j < n_blocks && ok; j++) {
            // the score buffer of block j+1 held block j-1, which the softmax threads left before they wrote P_{j-1}
            if (j + 1 < n_blocks) ok = scores(j + 1);
            ok = ok && mbar_wait(p_full, (uint32_t)j & 1u, abort_flag, status) && mbar_wait(v_full(pv.stage), pv.phase, abort_flag, status);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const uint64_t da = smem_desc_sw128(p_smem + half * (AT_TILE_BYTES / 2));
                const uint64_t db = smem_desc_sw128(v_smem(pv.stage) + half * (AT_TILE_BYTES / 2));
#pragma unroll
                for (int k = 0; k < AT_DBG_KSTEPS; k++) umma_bf16(tmem_o, da + 2u * k, db + 2u * k, idesc, (j | half | k) ? 1u : 0u);
            }
            umma_commit(v_empty(pv.stage));
            umma_commit(pv_done);
            pv.advance(AT_KV_STAGES);
        }
    } else if (warp >= 4) {
        // ---------------------------------------------------------- softmax: two threads per query row
        // Thread (row r, half hf) owns keys hf*64.. of every score block and, at the end, head
        // dimensions hf*64.. of the output.  The two threads of a row sit in different warps and
        // exchange their partial row maxima through shared memory at a named barrier; a thread whose
        // wait ran out marks `quit` and still joins that barrier, after which all of them leave.
        const int q4 = warp & 3, hf = (warp - 4) >> 2;
        const int r = q4 * 32 + lane;                                             // row inside the tile = TMEM lane
        const uint32_t lane_addr = ((uint32_t)(q4 * 32) << 16) + hf * 64;
        const float c = scale * 1.4426950408889634f;                              // scores to log2 units
        float m = 0.f, l = 0.f;
        bool alive = true;
#ifdef AT_DBG_CLOCK
        long long tk[8] = {0, 0, 0, 0, 0, 0, 0, 0}, tprev = clock64();
#endif
        for (int j = 0; j < n_blocks; j++) {
            const int b = j & 1;
            AT_TICK(0)
            if (alive) alive = mbar_wait(s_full(b), (uint32_t)(j >> 1) & 1u, abort_flag, status);
            alive = __all_sync(0xffffffffu, alive);
            AT_TICK(1)
            uint32_t sa[32], sb[32];                                              // this thread's 64 scores of the block
            float pmax = -CUDART_INF_F;
            if (alive) {
                tc_fence_after();
                tmem_ld32(tmem_base + b * 128 + lane_addr, sa);
                tmem_ld32(tmem_base + b * 128 + lane_addr + 32, sb);
                tmem_ld_wait();
                AT_TICK(2)
                if (j == n_blocks - 1) {                                          // the only block with keys after some of the rows
#pragma unroll
                    for (int i = 0; i < 32; i++) {
                        if (hf * 64 + i > r) sa[i] = 0xff800000u;
                        if (hf * 64 + 32 + i > r) sb[i] = 0xff800000u;
                    }
                }
                float mx[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
                for (int i = 0; i < 32; i += 4) {
                    mx[0] = max3(mx[0], __uint_as_float(sa[i]), __uint_as_float(sa[i + 1]));
                    mx[1] = max3(mx[1], __uint_as_float(sa[i + 2]), __uint_as_float(sa[i + 3]));
                    mx[2] = max3(mx[2], __uint_as_float(sb[i]), __uint_as_float(sb[i + 1]));
                    mx[3] = max3(mx[3], __uint_as_float(sb[i + 2]), __uint_as_float(sb[i + 3]));
                }
                pmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                xch[(b * 2 + hf) * 128 + r] = pmax;
            } else {
                *quit = 1;
            }
            AT_TICK(3)
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (*quit) break;
            AT_TICK(4)
            // every block holds at least one key the row may see (tiles and blocks are both cut from
            // the record's start in steps of 128), so the block maximum is finite
            const float bm = fmaxf(pmax, xch[(b * 2 + (hf ^ 1)) * 128 + r]) * c;
            float corr = 1.f;
            if (j == 0) m = bm;
            else if (bm > m + AT_LAZY) { corr = ex2_approx(m - bm); m = bm; l *= corr; }
            const bool rescale = __any_sync(0xffffffffu, corr != 1.f);
            // P = exp2(c s - m) as BF16 (values up to 2^8 while m lags the running maximum)
            uint32_t pk[32];
            float2 acc[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
            const float2 c2 = make_float2(c, c), nm2 = make_float2(-m, -m);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const uint32_t *src = i < 16 ? sa : sb;
                const float2 x = ffma2(make_float2(__uint_as_float(src[(2 * i) & 31]), __uint_as_float(src[(2 * i + 1) & 31])), c2, nm2);
#ifdef AT_DBG_NOEXP
                const float2 pp = make_float2(fminf(fmaxf(x.x, -1.f), 1.f) * 1e-3f + 2e-3f, fminf(fmaxf(x.y, -1.f), 1.f) * 1e-3f + 2e-3f);
#else
                const float2 pp = make_float2(ex2_approx(x.x), ex2_approx(x.y));
#endif
                acc[i & 1] = fadd2(acc[i & 1], pp);
                const __nv_bfloat162 bb = __floats2bfloat162_rn(pp.x, pp.y);
                pk[i] = *reinterpret_cast<const uint32_t *>(&bb);
            }
            const float sum = (acc[0].x + acc[1].x) + (acc[0].y + acc[1].y);
            l += sum;
            AT_TICK(5)
            // the P tile and the accumulator are free once the previous value product is done
            if (j > 0) alive = mbar_wait(pv_done, (uint32_t)(j - 1) & 1u, abort_flag, status);
            alive = __all_sync(0xffffffffu, alive);
            AT_TICK(6)
            if (!alive) continue;
            if (rescale) {
                tc_fence_after();
#pragma unroll
                for (int cc = 0; cc < 4; cc++) {                  // this warp's 32 rows, all 128 columns in two passes of two threads' halves
                    if ((cc >> 1) != hf) continue;                // each half of the row pair rescales its own 64 columns
                    uint32_t t32[32];
                    tmem_ld32(tmem_o + ((uint32_t)(q4 * 32) << 16) + cc * 32, t32);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; i++) t32[i] = __float_as_uint(__uint_as_float(t32[i]) * corr);
                    tmem_st32(tmem_o + ((uint32_t)(q4 * 32) << 16) + cc * 32, t32);
                }
                tmem_st_wait();
                tc_fence_before();
            }
            // swizzled K-major layout: this thread's 64 keys are one 128-byte row of its half tile,
            // chunk c8 of 8 keys at c8 ^ (r & 7)
            uint8_t *prow = smem_gen + AT_TILE_BYTES + hf * (AT_TILE_BYTES / 2) + r * 128;
#pragma unroll
            for (int c8 = 0; c8 < 8; c8++)
                *reinterpret_cast<uint4 *>(prow + ((c8 ^ (r & 7)) << 4)) = make_uint4(pk[c8 * 4], pk[c8 * 4 + 1], pk[c8 * 4 + 2], pk[c8 * 4 + 3]);
            tc_fence_before();
            fence_proxy_async_smem();
            mbar_arrive(p_full);
            AT_TICK(7)
        }
#ifdef AT_DBG_CLOCK
        if (blockIdx.x == gridDim.x - 1 && blockIdx.y == 0 && threadIdx.x == 128) {
            for (int k = 0; k < 8; k++) at_dbg[k] = (unsigned long long)tk[k];
            at_dbg[8] = (unsigned long long)n_blocks;
        }
#endif
        // the row's denominator is the sum of what its two threads added up (same reference maximum in both)
        if (alive) alive = mbar_wait(pv_done, (uint32_t)(n_blocks - 1) & 1u, abort_flag, status);
        if (!alive) *quit = 1;
        xch[((n_blocks & 1) * 2 + hf) * 128 + r] = l;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (!*quit) {
            tc_fence_after();
            const float lt = l + xch[((n_blocks & 1) * 2 + (hf ^ 1)) * 128 + r];
            const float inv = lt > 0.f ? 1.f / lt : 0.f;
            const int qg = tile.q0 + r;                                           // global token index of the row
            uint4 *dst = reinterpret_cast<uint4 *>(out + (long)qg * (NH * HD) + h * HD + hf * 64);
#pragma unroll
            for (int cc = 0; cc < 2; cc++) {
                uint32_t t32[32];
                tmem_ld32(tmem_o + lane_addr + cc * 32, t32);
                tmem_ld_wait();
                if (r < tile.q_len) {
#pragma unroll
                    for (int ch = 0; ch < 4; ch++) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const __nv_bfloat162 bb = __floats2bfloat162_rn(__uint_as_float(t32[ch * 8 + 2 * i]) * inv,
                                                                            __uint_as_float(t32[ch * 8 + 2 * i + 1]) * inv);
                            w[i] = *reinterpret_cast<const uint32_t *>(&bb);
                        }
                        dst[cc * 4 + ch] = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag && threadIdx.x == 0) {
        // a wait ran out: give loads already in flight a bounded chance to land
        for (int s = 0; s < 5; s++) {
            const int par = armed[s];
            if (par < 0) continue;
            const uint32_t bar = s == 0 ? q_full : s < 3 ? k_full(s - 1) : v_full(s - 3);
            const uint64_t t0 = globaltimer_ns();
            while (!mbar_try_wait(bar, (uint32_t)par) && globaltimer_ns() - t0 < 50000000ull) {}
        }
    }
    __syncthreads();
    if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, AT_TMEM_COLS); }
}

}  // namespace

extern "C" {

#ifdef AT_DBG_CLOCK
cudaError_t omni_attn_debug_read(unsigned long long *dst) { return cudaMemcpyFromSymbol(dst, at_dbg, sizeof(at_dbg)); }
#endif

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
