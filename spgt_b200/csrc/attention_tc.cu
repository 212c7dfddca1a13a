// Galerkin linear attention on the 5th-generation tensor cores (tcgen05, operands and accumulators in TMEM).
//
//   T[i][j]   = (1/S) * sum_s K[i][s] * V[j][s]        phase A: M = i, N = j, reduction over the grid nodes s
//   out[s][j] = sum_i Q[i][s] * T[i][j]                 phase B: M = s, N = j, reduction over i (dpk, zero padded to 40)
//
// Both contractions are 3xTF32 (x = hi + lo, three MMAs) so the result keeps fp32-level accuracy.  One cluster of
// 1-8 CTAs works on a (batch, head); each CTA streams its share of the S columns exactly once:
//   phase A  loader warps cp.async the raw K and V sub-tiles (32 columns) element-wise into 128B-swizzled K-major
//            shared memory (rows of Q/K/V are only 4-byte aligned, so no wider copy is legal); converter warps split
//            V in place into the hi / lo B operands and move the K rows - one row per thread - into TENSOR MEMORY as
//            the hi / lo A operands; one elected lane issues tcgen05.mma (128 x 48 x 8, A from TMEM, B from smem).
//            Rows / columns beyond dpk only produce accumulator entries that are never read.
//   reduce   the dpk x dpk partial sums of the cluster's CTAs are added in rank order through distributed shared
//            memory (deterministic, no global scratch), scaled by 1/S and written as the B operand of phase B.
//   phase B  128 threads own one grid node each: 34 coalesced loads of Q, split, tcgen05.st into TMEM (A operand);
//            the accumulator rows go back through shared memory and leave as coalesced stores.
// warps 0-3 loaders / Q producers, 4-7 converters / epilogue, 8-9 MMA issuers.  Two CTAs fit per SM (256 TMEM columns,
// ~102 KB shared memory each).  Every wait is a bounded mbarrier poll that records an error code on expiry.
#include "tc_common.cuh"

namespace spgt {

__device__ int g_attn_status = 0;

#ifdef SPGT_TC_TRACE
__device__ long long g_attn_trace[16 + 10 * 2048];
__device__ __forceinline__ long long at_gtime() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ int at_smid() { int t; asm volatile("mov.u32 %0, %%smid;" : "=r"(t)); return t; }
#define AT_TRACE(slot) do { if (blockIdx.x == 0) g_attn_trace[slot] = clock64(); \
    if (blockIdx.x < 2048) { g_attn_trace[16 + 10 * blockIdx.x + ((slot) & 7)] = at_gtime(); if ((slot) == 0) g_attn_trace[16 + 10 * blockIdx.x + 8] = at_smid(); } } while (0)
#else
#define AT_TRACE(slot) do { } while (0)
#endif

constexpr int AT_THREADS = 320;                 // warps 0-3 loaders, 4-7 converters, 8-9 MMA issuers
constexpr int AT_NP = 48;                       // N (and B-tile rows) padded to a multiple of 16
constexpr int AT_SUB = 32;                      // columns per phase-A stage
constexpr int AT_ST = 3;                        // phase-A stages
constexpr int AT_TILE = AT_NP * 128;            // one K-major operand image: 48 rows x 128 bytes
constexpr int AT_RAW_STAGE = 3 * AT_TILE;       // K raw | V hi (raw, split in place) | V lo
constexpr int AT_TB_OFF = AT_ST * AT_RAW_STAGE; // T images: [k-block 0 hi | lo | k-block 1 hi | lo]
constexpr int AT_OUT_OFF = AT_TB_OFF + 4 * AT_TILE;
constexpr int AT_OUT_BYTES = 4 * 32 * 36 * 4;
constexpr int AT_TC_OFF = AT_OUT_OFF + AT_OUT_BYTES;
constexpr int AT_TP = 36;                       // pitch of the dpk x dpk partial sums
constexpr int AT_BAR_OFF = AT_TC_OFF + AT_TP * AT_TP * 4;
constexpr int AT_SMEM_BYTES = 1024 + AT_BAR_OFF + 256;
constexpr int AT_TMEM_COLS = 256;
constexpr int AT_A1_COL = 96;                   // phase A: two accumulators at [0,48) and [48,96), two A stages (64 cols each) from here
constexpr int AT_A2_COL = 96;                   // phase B: accumulators at [0,48) and [48,96), A stages (80 cols) from here

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 2)
galerkin_attn_tc_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                        float* __restrict__ out, float* __restrict__ t_out, int S, int H, int merged) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* tb = smem + AT_TB_OFF;
    float* out_stage = reinterpret_cast<float*>(smem + AT_OUT_OFF);
    float* Tc = reinterpret_cast<float*>(smem + AT_TC_OFF);
    uint8_t* bar_mem = smem + AT_BAR_OFF;
    const uint32_t bars = smem_u32(bar_mem);
    auto raw_full = [&](int s) { return bars + 8u * s; };            // [3] loaders -> converters
    auto raw_empty = [&](int s) { return bars + 8u * (3 + s); };     // [3] MMA commit -> loaders
    auto ab_full = [&](int s) { return bars + 8u * (6 + s); };       // [3] converters -> MMA
    const uint32_t t_done = bars + 8u * 9;                           //     MMA commits -> T readout
    auto a_empty = [&](int s) { return bars + 8u * (18 + s); };      // [2] MMA commits -> converters (tensor-memory A stages)
    auto a2_full = [&](int s) { return bars + 8u * (10 + s); };      // [2] Q producers -> MMA
    auto a2_empty = [&](int s) { return bars + 8u * (12 + s); };     // [2] MMA commit -> Q producers
    auto d_full = [&](int b) { return bars + 8u * (14 + b); };       // [2] MMA commit -> epilogue
    auto d_empty = [&](int b) { return bars + 8u * (16 + b); };      // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mem + 192);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 200);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t C = cluster_nctarank();
    const uint32_t rank = cluster_ctarank();
    const int64_t bh = blockIdx.x / C;
    const float* Kg = K + bh * (int64_t)D * S;
    const float* Vg = V + bh * (int64_t)D * S;
    const float* Qg = Q + bh * (int64_t)D * S;

    const int nsub = (S + AT_SUB - 1) / AT_SUB;
    const int sub_begin = (int)(((int64_t)rank * nsub) / C);
    const int sub_end = (int)(((int64_t)(rank + 1) * nsub) / C);
    const int nmine = sub_end - sub_begin;

    if (tid == 0) {
        for (int s = 0; s < AT_ST; ++s) { mbar_init(raw_full(s), 128); mbar_init(raw_empty(s), 2); mbar_init(ab_full(s), 128); }
        mbar_init(t_done, 2);
        for (int s = 0; s < 2; ++s) mbar_init(a_empty(s), 2);
        for (int s = 0; s < 2; ++s) { mbar_init(a2_full(s), 128); mbar_init(a2_empty(s), 1); mbar_init(d_full(s), 1); mbar_init(d_empty(s), 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(AT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < 4 * AT_TILE / 16; i += AT_THREADS)            // K padding of the T images must be zero
        reinterpret_cast<uint4*>(tb)[i] = make_uint4(0u, 0u, 0u, 0u);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    constexpr uint32_t idesc = tc_idesc(AT_NP);

    if (tid == 0) AT_TRACE(0);
    // ============================== phase A: partial T over my columns ==============================
    if (warp < 4) {
        const int t = tid;
        for (int it = 0; it < nmine; ++it) {
            const uint32_t st = (uint32_t)(it % AT_ST), ph = (uint32_t)((it / AT_ST) & 1);
            if (!mbar_wait(raw_empty(st), ph ^ 1, abort_flag, 1, &g_attn_status)) break;
            const int s0 = (sub_begin + it) * AT_SUB;
            const uint32_t kdst = smem_base + st * AT_RAW_STAGE, vdst = kdst + AT_TILE;
#pragma unroll 3
            for (int e = t; e < D * AT_SUB; e += 128) {
                const int row = e >> 5, col = e & 31;
                const bool ok = s0 + col < S;
                const int64_t g = (int64_t)row * S + (ok ? s0 + col : 0);
                const uint32_t off = tc_swz(row, col >> 2) + (uint32_t)(col & 3) * 4u;
                const int n = ok ? 4 : 0;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(kdst + off), "l"(Kg + g), "r"(n) : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(vdst + off), "l"(Vg + g), "r"(n) : "memory");
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(raw_full(st)) : "memory");
        }
        cp_async_wait_all();
    } else if (warp < 8) {
        const int t = tid - 128, q = warp & 3;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const int krow = q * 32 + lane;                                 // K row moved to TMEM by this thread (q < 2)
        const bool k_warp = q * 32 < D;                                 // this warp owns at least one valid K row
        for (int it = 0; it < nmine; ++it) {
            const uint32_t st = (uint32_t)(it % AT_ST), ph = (uint32_t)((it / AT_ST) & 1);
            if (!mbar_wait(raw_full(st), ph, abort_flag, 2, &g_attn_status)) break;
            uint8_t* kraw = smem + st * AT_RAW_STAGE;
            uint8_t* vhi = kraw + AT_TILE;
            uint8_t* vlo = vhi + AT_TILE;
            // V: split the raw tile in place into the hi / lo B operands
            for (int e = t; e < D * 8; e += 128) {
                const uint32_t off = tc_swz(e >> 3, e & 7);
                const float4 v = *reinterpret_cast<const float4*>(vhi + off);
                uint32_t h[4], l[4];
                split_tf32_rn(v.x, h[0], l[0]); split_tf32_rn(v.y, h[1], l[1]); split_tf32_rn(v.z, h[2], l[2]); split_tf32_rn(v.w, h[3], l[3]);
                *reinterpret_cast<uint4*>(vhi + off) = make_uint4(h[0], h[1], h[2], h[3]);
                *reinterpret_cast<uint4*>(vlo + off) = make_uint4(l[0], l[1], l[2], l[3]);
            }
            // K: one row per thread into tensor memory, two stages there (freed by the MMAs two sub-tiles back).
            // Lanes beyond dpk move rows whose accumulator entries are never read.
            if (k_warp) {
                if (!mbar_wait(a_empty(it & 1), (uint32_t)(((it >> 1) & 1) ^ 1), abort_flag, 9, &g_attn_status)) break;
                tc_fence_after();
                const uint32_t a_hi = tmem_base + lane_addr + AT_A1_COL + (it & 1) * 64;
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 w = *reinterpret_cast<const float4*>(kraw + tc_swz(krow, 4 * h2 + j));
                        split_tf32_rn(w.x, hi[4 * j], lo[4 * j]); split_tf32_rn(w.y, hi[4 * j + 1], lo[4 * j + 1]);
                        split_tf32_rn(w.z, hi[4 * j + 2], lo[4 * j + 2]); split_tf32_rn(w.w, hi[4 * j + 3], lo[4 * j + 3]);
                    }
                    tc_st16(a_hi + 16 * h2, hi);
                    tc_st16(a_hi + 32 + 16 * h2, lo);
                }
                tc_wait_st();
                tc_fence_before();
            }
            fence_proxy_async();
            mbar_arrive(ab_full(st));
        }
    } else {
        // Two issuing warps (one thread issues an MMA only about every 54 cycles; a 128 x 48 x 8 MMA takes 24): warp 8
        // multiplies k-steps 0-1 of every sub-tile into the accumulator at column 0, warp 9 k-steps 2-3 into the one at
        // column 48; the two partial sums are added when T is read out.
        const int iw = warp - 8;
        const uint32_t d = tmem_base + (uint32_t)(iw * AT_NP);
        for (int it = 0; it < nmine; ++it) {
            const uint32_t st = (uint32_t)(it % AT_ST), ph = (uint32_t)((it / AT_ST) & 1);
            if (!mbar_wait(ab_full(st), ph, abort_flag, 3, &g_attn_status)) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t vhi = smem_base + st * AT_RAW_STAGE + AT_TILE;
                const uint64_t dbh = tc_smem_desc(vhi), dbl = tc_smem_desc(vhi + AT_TILE);
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    const int k8 = 2 * iw + kk;
                    const uint32_t ah = tmem_base + AT_A1_COL + (it & 1) * 64 + k8 * 8, al = ah + 32;
                    const uint64_t adv = (uint64_t)(k8 * 2);
                    tc_mma_tf32_ts(d, al, dbh + adv, idesc, (it > 0 || kk > 0) ? 1u : 0u);
                    tc_mma_tf32_ts(d, ah, dbl + adv, idesc, 1u);
                    tc_mma_tf32_ts(d, ah, dbh + adv, idesc, 1u);
                }
                tc_commit(raw_empty(st));
                tc_commit(a_empty(it & 1));
                if (it == nmine - 1) tc_commit(t_done);
            }
            __syncwarp();
        }
    }

    if (tid == 0) AT_TRACE(1);      // loaders done issuing
    if (tid == 128) AT_TRACE(2);    // converters done
    if (tid == 256) AT_TRACE(3);    // MMAs issued
    // ============================== reduce T over the cluster ==============================
    if (warp >= 4 && warp < 8) {
        const int q = warp & 3;
        if (q * 32 < D) {                                               // warps that hold valid rows of T
            float v[32], w[16];
            bool have = false;
            if (nmine > 0) have = mbar_wait(t_done, 0, abort_flag, 4, &g_attn_status);
            tc_fence_after();
            if (have) {
                float v2[32], w2[16];
                tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16), v);
                tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + 32, w);
                tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + AT_NP, v2);
                tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + AT_NP + 32, w2);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] += v2[j];
#pragma unroll
                for (int j = 0; j < 16; ++j) w[j] += w2[j];
            }
            const int row = q * 32 + lane;
            if (row < D) {
#pragma unroll
                for (int j = 0; j < 32; ++j) if (j < D) Tc[row * AT_TP + j] = have ? v[j] : 0.0f;
#pragma unroll
                for (int j = 0; j < 16; ++j) if (32 + j < D) Tc[row * AT_TP + 32 + j] = have ? w[j] : 0.0f;
            }
        }
    }
    tc_fence_before();
    cluster_sync_all();        // every CTA's Tc is complete; also a CTA-wide barrier (all threads arrive)
    tc_fence_after();
    {
        const float inv_s = 1.0f / (float)S;
        for (int e = tid; e < D * D; e += AT_THREADS) {
            const int i = e / D, j = e % D;
            float s = 0.0f;
            for (uint32_t r = 0; r < C; ++r) s += ld_dsmem_f32(Tc + i * AT_TP + j, r);
            s *= inv_s;
            if (t_out != nullptr && rank == 0) t_out[bh * D * D + e] = s;
            uint32_t hi, lo, lo2;
            split_tf32(s, hi, lo);
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo2) : "f"(__uint_as_float(lo)));
            // B operand of phase B: row j (N), k = i; k-block i / 32
            uint8_t* img = tb + (i >> 5) * (2 * AT_TILE);
            const uint32_t off = tc_swz(j, (i & 31) >> 2) + (uint32_t)(i & 3) * 4u;
            *reinterpret_cast<uint32_t*>(img + off) = hi;
            *reinterpret_cast<uint32_t*>(img + AT_TILE + off) = lo2;
        }
    }
    fence_proxy_async();
    __syncthreads();

    if (tid == 0) AT_TRACE(4);
    // ============================== phase B: out = Q^T T over my columns ==============================
    const int col_begin = sub_begin * AT_SUB;
    const int col_end = min(sub_end * AT_SUB, S);
    const int ntile = (col_end - col_begin + 127) / 128;
    const int64_t b_idx = bh / H, h_idx = bh % H;
    if (warp < 4) {
        const int q = warp & 3;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        for (int it = 0; it < ntile; ++it) {
            const uint32_t sa = (uint32_t)(it & 1), ph = (uint32_t)((it >> 1) & 1);
            const int s = col_begin + it * 128 + tid;
            const bool ok = s < col_end;
            float qv[40];
#pragma unroll
            for (int i = 0; i < 40; ++i) qv[i] = (i < D && ok) ? __ldg(Qg + (int64_t)i * S + s) : 0.0f;
            if (!mbar_wait(a2_empty(sa), ph ^ 1, abort_flag, 5, &g_attn_status)) break;
            tc_fence_after();
            const uint32_t a_hi = tmem_base + lane_addr + AT_A2_COL + sa * 80, a_lo = a_hi + 40;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) split_tf32_rn(qv[16 * c + j], hi[j], lo[j]);
                tc_st16(a_hi + 16 * c, hi);
                tc_st16(a_lo + 16 * c, lo);
            }
            {
                uint32_t hi[8], lo[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) split_tf32_rn(qv[32 + j], hi[j], lo[j]);
                tc_st8(a_hi + 32, hi);
                tc_st8(a_lo + 32, lo);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(a2_full(sa));
        }
    } else if (warp < 8) {
        const int q = warp & 3;
        float* os = out_stage + (warp - 4) * 32 * 36;
        for (int it = 0; it < ntile; ++it) {
            const uint32_t buf = (uint32_t)(it & 1), ph = (uint32_t)((it >> 1) & 1);
            if (!mbar_wait(d_full(buf), ph, abort_flag, 6, &g_attn_status)) break;
            tc_fence_after();
            float v[32], w[16];
            tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * AT_NP, v);
            tc_ld16(tmem_base + ((uint32_t)(q * 32) << 16) + buf * AT_NP + 32, w);
            tc_fence_before();
            mbar_arrive(d_empty(buf));                                  // the accumulator is in registers
#pragma unroll
            for (int j = 0; j < 32; ++j) if (j < D) os[lane * D + j] = v[j];
#pragma unroll
            for (int j = 0; j < 16; ++j) if (32 + j < D) os[lane * D + 32 + j] = w[j];
            __syncwarp();
            const int s0 = col_begin + it * 128 + q * 32;
            int nrows = col_end - s0;
            nrows = nrows > 32 ? 32 : nrows;
            if (nrows > 0) {
                if (!merged) {
                    float* dst = out + (bh * S + s0) * D;               // nrows * D contiguous floats
                    if constexpr (D % 2 == 0) {
                        for (int e = lane; e < nrows * D / 2; e += 32)
                            reinterpret_cast<float2*>(dst)[e] = reinterpret_cast<const float2*>(os)[e];
                    } else {
                        for (int e = lane; e < nrows * D; e += 32) dst[e] = os[e];
                    }
                } else {
                    float* dst = out + ((b_idx * S + s0) * H + h_idx) * D;   // row pitch H * D
                    if constexpr (D % 2 == 0) {
                        for (int e = lane; e < nrows * (D / 2); e += 32) {
                            const int r = e / (D / 2), c2 = e % (D / 2);
                            reinterpret_cast<float2*>(dst + (int64_t)r * H * D)[c2] = reinterpret_cast<const float2*>(os + r * D)[c2];
                        }
                    } else {
                        for (int e = lane; e < nrows * D; e += 32) dst[(int64_t)(e / D) * H * D + (e % D)] = os[e];
                    }
                }
            }
            __syncwarp();
        }
    } else if (warp == 8) {
        for (int it = 0; it < ntile; ++it) {
            const uint32_t sa = (uint32_t)(it & 1), ph = (uint32_t)((it >> 1) & 1);
            if (!mbar_wait(d_empty(sa), ph ^ 1, abort_flag, 7, &g_attn_status)) break;
            if (!mbar_wait(a2_full(sa), ph, abort_flag, 8, &g_attn_status)) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t d = tmem_base + sa * AT_NP;
#pragma unroll
                for (int k8 = 0; k8 < 5; ++k8) {
                    const uint32_t img = smem_base + AT_TB_OFF + (k8 >> 2) * (2 * AT_TILE);
                    const uint64_t adv = (uint64_t)((k8 & 3) * 2);
                    const uint64_t dbh = tc_smem_desc(img) + adv, dbl = tc_smem_desc(img + AT_TILE) + adv;
                    const uint32_t ah = tmem_base + AT_A2_COL + sa * 80 + k8 * 8, al = ah + 40;
                    tc_mma_tf32_ts(d, al, dbh, idesc, k8 > 0 ? 1u : 0u);
                    tc_mma_tf32_ts(d, ah, dbl, idesc, 1u);
                    tc_mma_tf32_ts(d, ah, dbh, idesc, 1u);
                }
                tc_commit(a2_empty(sa));
                tc_commit(d_full(sa));
            }
            __syncwarp();
        }
    }
    if (tid == 0) AT_TRACE(5);
    if (tid == 128) AT_TRACE(6);
    if (tid == 256) AT_TRACE(7);
    tc_fence_before();
    cluster_sync_all();        // keep Tc alive until every CTA of the cluster has read it; all tensor-memory work is done
    if (warp == 8) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(AT_TMEM_COLS) : "memory");
    }
}

template <int D>
static int launch_attn_tc_d(const float* Q, const float* K, const float* V, float* out, float* t_out, int64_t BH, int H,
                            int S, int merged, int cluster, cudaStream_t stream) {
    static bool configured = false;
    auto kern = galerkin_attn_tc_kernel<D>;
    if (!configured) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AT_SMEM_BYTES) != cudaSuccess) return launch_status();
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(BH * cluster), 1, 1);
    cfg.blockDim = dim3(AT_THREADS, 1, 1);
    cfg.dynamicSmemBytes = AT_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, Q, K, V, out, t_out, S, H, merged);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; (void)cudaGetLastError(); return SPGT_ERR_LAUNCH; }
    return launch_status();
}

int launch_attn_tc(const float* Q, const float* K, const float* V, float* out, float* t_out, int64_t BH, int H, int dpk,
                   int S, int merged, int cluster, cudaStream_t stream) {
    switch (dpk) {
        case 32: return launch_attn_tc_d<32>(Q, K, V, out, t_out, BH, H, S, merged, cluster, stream);
        case 33: return launch_attn_tc_d<33>(Q, K, V, out, t_out, BH, H, S, merged, cluster, stream);
        case 34: return launch_attn_tc_d<34>(Q, K, V, out, t_out, BH, H, S, merged, cluster, stream);
        default: return launch_attn_tc_d<35>(Q, K, V, out, t_out, BH, H, S, merged, cluster, stream);
    }
}

#ifdef SPGT_TC_TRACE
extern "C" int spgt_attn_trace_read(long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, g_attn_trace, sizeof(long long) * (16 + 10 * 2048)) == cudaSuccess ? 0 : SPGT_ERR_LAUNCH;
}
#endif

int attn_tc_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)) != cudaSuccess) return SPGT_ERR_LAUNCH;
    return v;
}

}  // namespace spgt
