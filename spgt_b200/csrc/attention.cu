// Galerkin linear attention for one (batch, head) per thread-block cluster, and the generic split-K
// batched skinny GEMM.
//
//   T[i][j]   = (1/S) * sum_s K[i][s] * V[j][s]        (dpk x dpk, reduction over all S grid nodes)
//   out[s][j] = sum_i Q[i][s] * T[i][j]
//
// HBM traffic is the algorithmic minimum: K, V and Q are each streamed once, out is written once; the dpk x dpk
// partial sums of the CTAs that share a (batch, head) are combined through distributed shared memory inside a
// cluster, in rank order, so there is no global scratch and the result is bitwise reproducible.
// Both contractions run on the tensor cores as 3xTF32 (fp32-level accuracy); dpk = 34 = 2 position rows + 32
// channels is covered with 16x8 MMA tiles whose last row/column tile is shifted to end at dpk (overlapping the
// previous tile) instead of being zero padded.
//
// Every warp owns a private double-buffered cp.async pipeline over 32-column sub-tiles, so the main loops contain
// no block-wide barrier.
#include "common.cuh"

namespace spgt {

constexpr int ATT_WARPS = 4;
constexpr int ATT_THREADS = ATT_WARPS * 32;
constexpr int ATT_SUB = 32;          // columns (grid nodes) per warp sub-tile
constexpr int ATT_KP = ATT_SUB + 4;  // K/V tile pitch: == 4 (mod 32) -> conflict-free A/B fragment loads
constexpr int ATT_QP = 40;           // Q tile and T pitch: == 8 (mod 32)
constexpr int ATT_TP = 36;           // pitch of the dpk x dpk partial sums

template <int D> struct AttnSmem {
    static constexpr int KV_STAGE = 2 * D * ATT_KP;                  // floats: K tile then V tile
    static constexpr int WARP_FLOATS = 2 * KV_STAGE;                 // two stages
    static constexpr int Q_STAGE = ATT_QP * ATT_QP;                  // [40 k-rows][40]
    static constexpr int OS_OFF = 2 * Q_STAGE;                       // output staging [32][D]
    static constexpr int TW_OFF = WARP_FLOATS - ATT_TP * ATT_TP;     // warp partial of T at the end of the region
    static_assert(OS_OFF + 32 * D <= WARP_FLOATS, "phase-B buffers must fit in the warp region");
    static_assert(TW_OFF >= 2 * Q_STAGE, "warp partial must not overlap the prefetched Q stage");
    static constexpr int THI_OFF = ATT_WARPS * WARP_FLOATS;
    static constexpr int TLO_OFF = THI_OFF + ATT_QP * ATT_QP;
    static constexpr int TC_OFF = TLO_OFF + ATT_QP * ATT_QP;
    static constexpr int TOTAL_FLOATS = TC_OFF + ATT_TP * ATT_TP;
    static constexpr size_t BYTES = (size_t)TOTAL_FLOATS * sizeof(float);
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 2)
galerkin_attn_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                     float* __restrict__ out, float* __restrict__ t_out, int S, int H, int merged) {
    constexpr int MT = (D + 15) / 16;           // 16-row tiles over dpk (last one shifted to end at D)
    constexpr int NT = (D + 7) / 8;             // 8-column tiles over dpk (last one shifted)
    constexpr int KS = (D + 7) / 8;             // k-steps of phase B (zero padded up to 8*KS)
    using L = AttnSmem<D>;
    extern __shared__ __align__(16) float smem[];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t C = cluster_nctarank();
    const uint32_t rank = cluster_ctarank();
    const int64_t bh = blockIdx.x / C;
    const float* Kg = K + bh * (int64_t)D * S;
    const float* Vg = V + bh * (int64_t)D * S;
    const float* Qg = Q + bh * (int64_t)D * S;

    float* wreg = smem + warp * L::WARP_FLOATS;
    float* Thi = smem + L::THI_OFF;
    float* Tlo = smem + L::TLO_OFF;
    float* Tc = smem + L::TC_OFF;

    // this CTA's contiguous range of sub-tiles, dealt round-robin to its warps
    const int nsub = (S + ATT_SUB - 1) / ATT_SUB;
    const int sub_begin = (int)(((int64_t)rank * nsub) / C);
    const int sub_end = (int)(((int64_t)(rank + 1) * nsub) / C);
    const int nmine = (sub_end - sub_begin - warp + ATT_WARPS - 1) / ATT_WARPS;   // may be <= 0

    int m0[MT], n0[NT];
#pragma unroll
    for (int i = 0; i < MT; ++i) m0[i] = (i == MT - 1) ? D - 16 : 16 * i;
#pragma unroll
    for (int i = 0; i < NT; ++i) n0[i] = (i == NT - 1) ? D - 8 : 8 * i;

    // ------------------------------ phase A: partial T over my columns ------------------------------
    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0f;

    auto load_kv = [&](int it, int stage) {
        const int col = (sub_begin + warp + it * ATT_WARPS) * ATT_SUB + lane;
        const bool ok = col < S;
        const int64_t c = ok ? col : S - 1;
        float* kb = wreg + stage * L::KV_STAGE + lane;
        float* vb = kb + D * ATT_KP;
        const float* kp = Kg + c;
        const float* vp = Vg + c;
#pragma unroll 2
        for (int i = 0; i < D; ++i) {
            cp_async_zfill<4>(kb + i * ATT_KP, kp + (int64_t)i * S, ok);
            cp_async_zfill<4>(vb + i * ATT_KP, vp + (int64_t)i * S, ok);
        }
        cp_async_commit();
    };

    if (nmine > 0) load_kv(0, 0);
    for (int it = 0; it < nmine; ++it) {
        if (it + 1 < nmine) {
            load_kv(it + 1, (it + 1) & 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        const float* kb = wreg + (it & 1) * L::KV_STAGE;
        const float* vb = kb + D * ATT_KP;
#pragma unroll
        for (int k8 = 0; k8 < ATT_SUB / 8; ++k8) {
            const int kk = k8 * 8 + t;
            uint32_t ahi[MT][4], alo[MT][4];
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const float* p = kb + (m0[i] + g) * ATT_KP + kk;
                split_tf32(p[0], ahi[i][0], alo[i][0]);
                split_tf32(p[8 * ATT_KP], ahi[i][1], alo[i][1]);
                split_tf32(p[4], ahi[i][2], alo[i][2]);
                split_tf32(p[8 * ATT_KP + 4], ahi[i][3], alo[i][3]);
            }
            uint32_t bhi[NT][2], blo[NT][2];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const float* p = vb + (n0[j] + g) * ATT_KP + kk;
                split_tf32(p[0], bhi[j][0], blo[j][0]);
                split_tf32(p[4], bhi[j][1], blo[j][1]);
            }
            // three passes over all tiles: consecutive MMAs never touch the same accumulator
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_tf32(acc[i][j], alo[i], bhi[j]);
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_tf32(acc[i][j], ahi[i], blo[j]);
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_tf32(acc[i][j], ahi[i], bhi[j]);
        }
        __syncwarp();
    }

    // Prefetch the first Q sub-tile (phase B) so that it overlaps the reductions; zero the k-padding rows first.
    auto load_q = [&](int it, int stage) {
        const int col = (sub_begin + warp + it * ATT_WARPS) * ATT_SUB + lane;
        const bool ok = col < S;
        const float* qp = Qg + (ok ? col : S - 1);
        float* qb = wreg + stage * L::Q_STAGE + lane;
#pragma unroll 2
        for (int i = 0; i < D; ++i) cp_async_zfill<4>(qb + i * ATT_QP, qp + (int64_t)i * S, ok);
        cp_async_commit();
    };
    for (int i = lane; i < 2 * L::Q_STAGE; i += 32) {
        const int row = (i % L::Q_STAGE) / ATT_QP;
        if (row >= D) wreg[i] = 0.0f;
    }
    __syncwarp();
    if (nmine > 0) load_q(0, 0);

    // warp partial -> shared (each (i,j) written by exactly one tile), then CTA sum in warp order
    {
        float* Tw = wreg + L::TW_OFF;
#pragma unroll
        for (int i = 0; i < MT; ++i)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int lo_r = (i == MT - 1) ? 16 * (MT - 1) : 0;    // rows below this index belong to tile i-1
                const int lo_c = (j == NT - 1) ? 8 * (NT - 1) : 0;
                const int r0 = m0[i] + g, c0 = n0[j] + 2 * t;
                if (r0 >= lo_r) {
                    if (c0 >= lo_c) Tw[r0 * ATT_TP + c0] = acc[i][j][0];
                    if (c0 + 1 >= lo_c) Tw[r0 * ATT_TP + c0 + 1] = acc[i][j][1];
                }
                if (r0 + 8 >= lo_r) {
                    if (c0 >= lo_c) Tw[(r0 + 8) * ATT_TP + c0] = acc[i][j][2];
                    if (c0 + 1 >= lo_c) Tw[(r0 + 8) * ATT_TP + c0 + 1] = acc[i][j][3];
                }
            }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < D * D; e += ATT_THREADS) {
        const int o = (e / D) * ATT_TP + (e % D);
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < ATT_WARPS; ++w) s += smem[w * L::WARP_FLOATS + L::TW_OFF + o];
        Tc[o] = s;
    }
    for (int e = threadIdx.x; e < 2 * ATT_QP * ATT_QP; e += ATT_THREADS) Thi[e] = 0.0f;   // Thi and Tlo are adjacent
    cluster_sync_all();   // every CTA's Tc is complete and visible cluster-wide (also orders the zero fill above)

    const float inv_s = 1.0f / (float)S;
    for (int e = threadIdx.x; e < D * D; e += ATT_THREADS) {
        const int i = e / D, j = e % D;
        float s = 0.0f;
        for (uint32_t r = 0; r < C; ++r) s += ld_dsmem_f32(Tc + i * ATT_TP + j, r);
        s *= inv_s;
        if (t_out != nullptr && rank == 0) t_out[bh * D * D + e] = s;
        uint32_t hi, lo;
        split_tf32(s, hi, lo);
        Thi[i * ATT_QP + j] = __uint_as_float(hi);
        Tlo[i * ATT_QP + j] = __uint_as_float(lo);
    }
    __syncthreads();

    // ------------------------------ phase B: out = Q^T T over my columns ------------------------------
    const int64_t b_idx = bh / H, h_idx = bh % H;
    for (int it = 0; it < nmine; ++it) {
        if (it + 1 < nmine) {
            load_q(it + 1, (it + 1) & 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        const float* qb = wreg + (it & 1) * L::Q_STAGE;
        float o[2][NT][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int r = 0; r < 4; ++r) o[i][j][r] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int kr = ks * 8 + t;
            uint32_t ahi[2][4], alo[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float* p = qb + kr * ATT_QP + 16 * i + g;
                split_tf32(p[0], ahi[i][0], alo[i][0]);
                split_tf32(p[8], ahi[i][1], alo[i][1]);
                split_tf32(p[4 * ATT_QP], ahi[i][2], alo[i][2]);
                split_tf32(p[4 * ATT_QP + 8], ahi[i][3], alo[i][3]);
            }
            uint32_t bhi[NT][2], blo[NT][2];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int off = kr * ATT_QP + n0[j] + g;
                bhi[j][0] = __float_as_uint(Thi[off]);
                bhi[j][1] = __float_as_uint(Thi[off + 4 * ATT_QP]);
                blo[j][0] = __float_as_uint(Tlo[off]);
                blo[j][1] = __float_as_uint(Tlo[off + 4 * ATT_QP]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_tf32(o[i][j], alo[i], bhi[j]);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_tf32(o[i][j], ahi[i], blo[j]);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_tf32(o[i][j], ahi[i], bhi[j]);
        }
        // stage the 32 x D tile in shared memory in the global row-major order, then store coalesced
        float* os = wreg + L::OS_OFF;
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int lo_c = (j == NT - 1) ? 8 * (NT - 1) : 0;
                const int r0 = 16 * i + g, c0 = n0[j] + 2 * t;
                if (c0 >= lo_c) { os[r0 * D + c0] = o[i][j][0]; os[(r0 + 8) * D + c0] = o[i][j][2]; }
                if (c0 + 1 >= lo_c) { os[r0 * D + c0 + 1] = o[i][j][1]; os[(r0 + 8) * D + c0 + 1] = o[i][j][3]; }
            }
        __syncwarp();
        const int s0 = (sub_begin + warp + it * ATT_WARPS) * ATT_SUB;
        const int rows = min(ATT_SUB, S - s0);
        if (!merged) {
            float* dst = out + (bh * S + s0) * D;           // rows*D contiguous floats
            if constexpr (D % 2 == 0) {
                for (int e = lane; e < rows * D / 2; e += 32)
                    reinterpret_cast<float2*>(dst)[e] = reinterpret_cast<const float2*>(os)[e];
            } else {
                for (int e = lane; e < rows * D; e += 32) dst[e] = os[e];
            }
        } else {
            float* dst = out + ((b_idx * S + s0) * H + h_idx) * D;   // row pitch H*D
            if constexpr (D % 2 == 0) {
                for (int e = lane; e < rows * (D / 2); e += 32) {
                    const int r = e / (D / 2), c2 = e % (D / 2);
                    reinterpret_cast<float2*>(dst + (int64_t)r * H * D)[c2] = reinterpret_cast<const float2*>(os + r * D)[c2];
                }
            } else {
                for (int e = lane; e < rows * D; e += 32) dst[(int64_t)(e / D) * H * D + (e % D)] = os[e];
            }
        }
        __syncwarp();
    }
    cluster_sync_all();   // keep Tc alive until every CTA of the cluster has read it
}

// ------------------------------------------------------------------------------------------------------------
// Generic batched skinny GEMM  C[b] = alpha * A[b] (M x K) * B[b] (K x N), K long: split-K, two passes.
// Pass 1: one CTA per (batch, 32x32 output tile, split) writes its partial tile to the workspace.
// Pass 2: partial tiles are summed in split order and scaled.
// ------------------------------------------------------------------------------------------------------------
constexpr int SK_WARPS = 4;
constexpr int SK_AP = 36;   // A tile [32 m][32 k], pitch == 4 (mod 32)
constexpr int SK_BP = 40;   // B tile [32 k][32 n], pitch == 8 (mod 32)
constexpr int SK_STAGE = 32 * SK_AP + 32 * SK_BP;
constexpr int SK_WARP_FLOATS = 2 * SK_STAGE;

__global__ void __launch_bounds__(SK_WARPS * 32, 4)
skinny_splitk_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ ws,
                     int M, int N, int K, int tiles_n, int tiles, int splits, int vecB) {
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int split = blockIdx.x % splits;
    const int tile = (blockIdx.x / splits) % tiles;
    const int64_t b = blockIdx.x / ((int64_t)splits * tiles);
    const int tm = tile / tiles_n, tn = tile % tiles_n;
    const float* Ag = A + b * (int64_t)M * K;
    const float* Bg = B + b * (int64_t)K * N;
    float* wreg = smem + warp * SK_WARP_FLOATS;

    const int nsub = (K + 31) / 32;
    const int sub_begin = (int)(((int64_t)split * nsub) / splits);
    const int sub_end = (int)(((int64_t)(split + 1) * nsub) / splits);
    const int nmine = (sub_end - sub_begin - warp + SK_WARPS - 1) / SK_WARPS;

    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0f;

    auto load = [&](int it, int stage) {
        const int k0 = (sub_begin + warp + it * SK_WARPS) * 32;
        float* as = wreg + stage * SK_STAGE;
        float* bs = as + 32 * SK_AP;
        {   // A: lane <-> k, rows m
            const int k = k0 + lane;
            const bool kok = k < K;
            const float* ap = Ag + (kok ? k : K - 1);
#pragma unroll 4
            for (int i = 0; i < 32; ++i) {
                const int m = tm * 32 + i;
                const bool ok = kok && m < M;
                cp_async_zfill<4>(as + i * SK_AP + lane, ap + (int64_t)(ok ? m : 0) * K, ok);
            }
        }
        if (vecB) {   // B rows are 16-byte aligned: lane <-> (row within 4, float4 within row)
            const int r4 = lane >> 3, c4 = (lane & 7) * 4;
            const int n = tn * 32 + c4;
#pragma unroll 4
            for (int i = 0; i < 8; ++i) {
                const int k = k0 + i * 4 + r4;
                const bool ok = k < K && n < N;          // N % 4 == 0 here, so a float4 is all-in or all-out
                cp_async_zfill<16>(bs + (i * 4 + r4) * SK_BP + c4, Bg + (int64_t)(ok ? k : 0) * N + (ok ? n : 0), ok);
            }
        } else {      // lane <-> n
            const int n = tn * 32 + lane;
            const bool nok = n < N;
#pragma unroll 4
            for (int i = 0; i < 32; ++i) {
                const int k = k0 + i;
                const bool ok = nok && k < K;
                cp_async_zfill<4>(bs + i * SK_BP + lane, Bg + (int64_t)(ok ? k : 0) * N + (ok ? n : 0), ok);
            }
        }
        cp_async_commit();
    };

    if (nmine > 0) load(0, 0);
    for (int it = 0; it < nmine; ++it) {
        if (it + 1 < nmine) {
            load(it + 1, (it + 1) & 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        const float* as = wreg + (it & 1) * SK_STAGE;
        const float* bs = as + 32 * SK_AP;
#pragma unroll
        for (int k8 = 0; k8 < 4; ++k8) {
            const int kk = k8 * 8 + t;
            uint32_t ahi[2][4], alo[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float* p = as + (16 * i + g) * SK_AP + kk;
                split_tf32(p[0], ahi[i][0], alo[i][0]);
                split_tf32(p[8 * SK_AP], ahi[i][1], alo[i][1]);
                split_tf32(p[4], ahi[i][2], alo[i][2]);
                split_tf32(p[8 * SK_AP + 4], ahi[i][3], alo[i][3]);
            }
            uint32_t bhi[4][2], blo[4][2];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* p = bs + kk * SK_BP + 8 * j + g;
                split_tf32(p[0], bhi[j][0], blo[j][0]);
                split_tf32(p[4 * SK_BP], bhi[j][1], blo[j][1]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_tf32(acc[i][j], alo[i], bhi[j]);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_tf32(acc[i][j], ahi[i], blo[j]);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_tf32(acc[i][j], ahi[i], bhi[j]);
        }
        __syncwarp();
    }
    // warp partial -> shared [32][32], CTA sum in warp order -> workspace
    float* tw = wreg;   // 1024 floats, all loads of this warp have completed
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int r0 = 16 * i + g, c0 = 8 * j + 2 * t;
            tw[r0 * 32 + c0] = acc[i][j][0];
            tw[r0 * 32 + c0 + 1] = acc[i][j][1];
            tw[(r0 + 8) * 32 + c0] = acc[i][j][2];
            tw[(r0 + 8) * 32 + c0 + 1] = acc[i][j][3];
        }
    __syncthreads();
    float* dst = ws + (((b * tiles + tile) * splits) + split) * 1024;
    for (int e = threadIdx.x; e < 1024; e += SK_WARPS * 32) {
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) s += smem[w * SK_WARP_FLOATS + e];
        dst[e] = s;
    }
}

__global__ void __launch_bounds__(256)
skinny_reduce_kernel(const float* __restrict__ ws, float* __restrict__ C, float alpha, int M, int N, int tiles_n,
                     int tiles, int splits) {
    const int tile = blockIdx.x % tiles;
    const int64_t b = blockIdx.x / tiles;
    const int tm = tile / tiles_n, tn = tile % tiles_n;
    const float* src = ws + ((b * tiles + tile) * splits) * 1024;
    for (int e = threadIdx.x; e < 1024; e += 256) {
        float s = 0.0f;
        for (int sp = 0; sp < splits; ++sp) s += src[(int64_t)sp * 1024 + e];
        const int m = tm * 32 + e / 32, n = tn * 32 + e % 32;
        if (m < M && n < N) C[b * (int64_t)M * N + (int64_t)m * N + n] = alpha * s;
    }
}

// ------------------------------------------------------------------------------------------------------------
// The same product in ONE launch with the k range of all (batch, tile) items cut evenly over one persistent CTA
// per SM ("stream-K"): the items' 16-wide k slices form one long list, CTA c takes the c-th equal share of it, so a
// CTA works on the end of one item, possibly some whole items, and the start of another.  An item that lies
// inside one CTA is scaled and stored directly.  The pieces of an item that spans several CTAs go to a small
// scratch (two 32x32 slots per CTA); every CTA that finishes a piece takes a ticket on the item's counter and the
// one that takes the last ticket adds the pieces in CTA order - a fixed order, so the result is bit-identical from
// run to run - scales the sum and stores it.  Nothing ever waits for another CTA.
// Rows of A are only 4-byte aligned (K is arbitrary): a row piece is fetched as five 16-byte cp.async chunks that
// start at the aligned element at or below its first column; the wanted elements then sit (element index of the
// piece start) mod 4 floats into the shared-memory row.  Requires N % 4 == 0 (16-byte chunks of the B rows).
// ------------------------------------------------------------------------------------------------------------
// The kernel is bound by latency, not by a pipe (measured with 6 warps per SM: tensor pipe 33 %, issue slots 35 %, DRAM 41 %
// busy, top stall "wait"), so the slices are 16 wide: a warp's three-stage ring takes 15 KB and twelve warps fit an SM.
constexpr int SKS_WARPS = 12, SKS_STAGES = 3;
constexpr int SKS_K = 16;    // k slice of one stage
constexpr int SKS_AP = 20;   // A tile row: 16 wanted floats + up to 3 of shift, five 16-byte chunks; rows 20 floats apart: conflict-free fragments
constexpr int SKS_BP = 40;   // B tile row pitch, == 8 (mod 32)
constexpr int SKS_STAGE = 32 * SKS_AP + SKS_K * SKS_BP;
constexpr int SKS_WARP_FLOATS = SKS_STAGES * SKS_STAGE;
constexpr size_t SKS_SMEM = (size_t)SKS_WARPS * SKS_WARP_FLOATS * sizeof(float);
static_assert(SKS_WARP_FLOATS >= 1024, "a warp's region also holds its 32x32 partial tile");

struct SksPlan { int64_t total; int nsub; int tiles, tiles_n; int P; };
// CTA that owns unit u of the list: the c with floor(c * total / P) <= u < floor((c + 1) * total / P)
__host__ __device__ inline int sks_owner(int64_t u, int64_t total, int P) { return (int)(((u + 1) * P - 1) / total); }

__global__ void __launch_bounds__(SKS_WARPS * 32, 1)
skinny_streamk_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, float alpha,
                      int M, int N, int K, SksPlan pl, float* __restrict__ pieces, unsigned int* __restrict__ tickets) {
    extern __shared__ __align__(16) float smem[];
    __shared__ int s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int c = blockIdx.x, P = pl.P, nsub = pl.nsub;
    const int64_t u_begin = ((int64_t)c * pl.total) / P, u_end = ((int64_t)(c + 1) * pl.total) / P;
    float* wreg = smem + warp * SKS_WARP_FLOATS;

    for (int64_t u0 = u_begin; u0 < u_end;) {
        const int64_t item = u0 / nsub;
        const int sub0 = (int)(u0 - item * nsub);
        const int sub1 = (int)((u_end - item * nsub) < nsub ? (u_end - item * nsub) : nsub);     // this CTA's slices [sub0, sub1) of the item
        const int tile = (int)(item % pl.tiles);
        const int64_t b = item / pl.tiles;
        const int tm = tile / pl.tiles_n, tn = tile % pl.tiles_n;
        const float* Bg = B + b * (int64_t)K * N;
        const int64_t a_row0 = (b * M + (int64_t)tm * 32) * K;          // element index of A[b][tm * 32][0]
        const int nmine = (sub1 - sub0 - warp + SKS_WARPS - 1) / SKS_WARPS;

        int a_sh[2][2];                                                  // shift of rows 16 i + g and 16 i + g + 8
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int h = 0; h < 2; ++h) a_sh[i][h] = (int)((a_row0 + (int64_t)(16 * i + g + 8 * h) * K) & 3);

        // What a thread copies is the same for every slice but for the k offset, so the per-chunk values are computed once per
        // item: the aligned source of A chunk idx = lane + 32 n -> (row, chunk in row) at this warp's first slice, and the
        // elements from there to the end of the row (0 for rows beyond M).  This warp's slices are SKS_WARPS * SKS_K apart, a
        // multiple of four elements, so the alignment shift of a row is the same in every slice.  (The address arithmetic was
        // 40 % of the instructions of a slice.)
        const int k00 = (sub0 + warp) * SKS_K;
        const float* a_src[5];
        int a_rem[5];
        uint32_t a_dst[5];
#pragma unroll
        for (int n = 0; n < 5; ++n) {
            const int idx = lane + 32 * n, row = idx / 5, ch = idx - 5 * row;
            const int64_t e = a_row0 + (int64_t)row * K + k00;           // element index of the first wanted element
            const int64_t start = (e & ~(int64_t)3) + 4 * ch;
            int64_t rem = (tm * 32 + row < M) ? (a_row0 + (int64_t)row * K + K - start) : 0;
            rem = rem < 0 ? 0 : (rem > 0x7fffffff ? 0x7fffffff : rem);
            a_src[n] = A + start; a_rem[n] = (int)rem; a_dst[n] = (uint32_t)((row * SKS_AP + 4 * ch) * 4);
        }
        const int b_r4 = lane >> 3, b_c4 = (lane & 7) * 4;
        const bool b_col_ok = tn * 32 + b_c4 < N;                        // N % 4 == 0: a chunk is all inside or all outside
        const float* b_src = Bg + (int64_t)(k00 + b_r4) * N + (b_col_ok ? tn * 32 + b_c4 : 0);
        auto load = [&](int it, int stage) {
            const int koff = it * (SKS_WARPS * SKS_K);
            float* as = wreg + stage * SKS_STAGE;
            float* bs = as + 32 * SKS_AP;
            const uint32_t as_u = smem_u32(as);
#pragma unroll
            for (int n = 0; n < 5; ++n) {
                int valid = a_rem[n] - koff;
                valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(as_u + a_dst[n]),
                             "l"(valid > 0 ? a_src[n] + koff : A), "r"(valid * 4) : "memory");
            }
#pragma unroll
            for (int i = 0; i < SKS_K / 4; ++i) {
                const bool ok = b_col_ok && k00 + koff + i * 4 + b_r4 < K;
                cp_async_zfill<16>(bs + (i * 4 + b_r4) * SKS_BP + b_c4, ok ? b_src + (int64_t)(koff + i * 4) * N : Bg, ok);
            }
            cp_async_commit();
        };

        // Two levels of accumulation: the tensor cores add into `acc` for sixteen slices (96 MMAs per element), then `acc` is
        // added to `tot` with ordinary fp32 additions.  The accumulate step of an MMA truncates, so the error of one long
        // chain grows with its length; short chains keep sums of 10^4 .. 10^5 cancelling terms at fp32 accuracy.
        float acc[2][4][4], tot[2][4][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int q = 0; q < 4; ++q) { acc[i][j][q] = 0.0f; tot[i][j][q] = 0.0f; }

        if (nmine > 0) load(0, 0);
        if (nmine > 1) load(1, 1);
        for (int it = 0; it < nmine; ++it) {
            if ((it & 15) == 0 && it > 0) {
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int q = 0; q < 4; ++q) { tot[i][j][q] += acc[i][j][q]; acc[i][j][q] = 0.0f; }
            }
            if (it + 2 < nmine) { load(it + 2, (it + 2) % SKS_STAGES); cp_async_wait<2>(); }
            else if (it + 1 < nmine) cp_async_wait<1>();
            else cp_async_wait<0>();
            __syncwarp();
            const float* as = wreg + (it % SKS_STAGES) * SKS_STAGE;
            const float* bs = as + 32 * SKS_AP;
#pragma unroll
            for (int k8 = 0; k8 < SKS_K / 8; ++k8) {
                const int kk = k8 * 8 + t;
                uint32_t ahi[2][4], alo[2][4];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const float* p0 = as + (16 * i + g) * SKS_AP + kk + a_sh[i][0];
                    const float* p1 = as + (16 * i + g + 8) * SKS_AP + kk + a_sh[i][1];
                    split_tf32(p0[0], ahi[i][0], alo[i][0]);
                    split_tf32(p1[0], ahi[i][1], alo[i][1]);
                    split_tf32(p0[4], ahi[i][2], alo[i][2]);
                    split_tf32(p1[4], ahi[i][3], alo[i][3]);
                }
                uint32_t bhi[4][2], blo[4][2];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float* p = bs + kk * SKS_BP + 8 * j + g;
                    split_tf32(p[0], bhi[j][0], blo[j][0]);
                    split_tf32(p[4 * SKS_BP], bhi[j][1], blo[j][1]);
                }
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_tf32(acc[i][j], alo[i], bhi[j]);
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_tf32(acc[i][j], ahi[i], blo[j]);
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_tf32(acc[i][j], ahi[i], bhi[j]);
            }
            __syncwarp();
        }
        // warp partial -> shared [32][32] (all copies of this warp have landed and been read), CTA sum in warp order
        float* tw = wreg;
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int r0 = 16 * i + g, c0 = 8 * j + 2 * t;
                tw[r0 * 32 + c0] = tot[i][j][0] + acc[i][j][0];
                tw[r0 * 32 + c0 + 1] = tot[i][j][1] + acc[i][j][1];
                tw[(r0 + 8) * 32 + c0] = tot[i][j][2] + acc[i][j][2];
                tw[(r0 + 8) * 32 + c0 + 1] = tot[i][j][3] + acc[i][j][3];
            }
        __syncthreads();
        const bool whole = sub0 == 0 && sub1 == nsub;                    // the item lies inside this CTA
        const int c_first = sks_owner(item * nsub, pl.total, P), c_last = sks_owner((item + 1) * nsub - 1, pl.total, P);
        float* piece = pieces + ((int64_t)2 * c + (c == c_first ? 1 : 0)) * 1024;
        float* Cb = C + b * (int64_t)M * N;
        for (int e = threadIdx.x; e < 1024; e += SKS_WARPS * 32) {
            float sum = 0.0f;
#pragma unroll
            for (int w = 0; w < SKS_WARPS; ++w) sum += smem[w * SKS_WARP_FLOATS + e];
            if (whole) {
                const int m = tm * 32 + e / 32, n = tn * 32 + e % 32;
                if (m < M && n < N) Cb[(int64_t)m * N + n] = alpha * sum;
            } else {
                __stcg(piece + e, sum);
            }
        }
        if (!whole) {
            __threadfence();                                             // this thread's piece elements are visible device-wide
            __syncthreads();
            if (threadIdx.x == 0) {
                const unsigned int ticket = atomicAdd(tickets + c_first, 1u);
                s_last = (ticket == (unsigned int)(c_last - c_first)) ? 1 : 0;
            }
            __syncthreads();
            if (s_last) {                                                // every piece of the item has been written
                __threadfence();
                for (int e = threadIdx.x; e < 1024; e += SKS_WARPS * 32) {
                    float sum = 0.0f;
                    for (int cc = c_first; cc <= c_last; ++cc)
                        sum += __ldcg(pieces + ((int64_t)2 * cc + (cc == c_first ? 1 : 0)) * 1024 + e);
                    const int m = tm * 32 + e / 32, n = tn * 32 + e % 32;
                    if (m < M && n < N) Cb[(int64_t)m * N + n] = alpha * sum;
                }
                if (threadIdx.x == 0) tickets[c_first] = 0u;             // ready for the next call
            }
        }
        __syncthreads();                                                 // the warp regions are reused by the next item
        u0 = item * nsub + sub1;
    }
}

static SmemOptIn g_skinny_smem;           // shared-memory opt-in of skinny_splitk_kernel, per device
static int g_attn_cluster_override = 0;   // 0 = heuristic; set through spgt_set_tuning("attn_cluster", n)
static int g_attn_impl = 0;               // 0 = tcgen05 kernel (attention_tc.cu, default), 1 = warp-MMA kernel of this file

// defined in attention_tc.cu
int launch_attn_tc(const float* Q, const float* K, const float* V, float* out, float* t_out, int64_t BH, int H, int dpk,
                   int S, int merged, int cluster, cudaStream_t stream);

void spectral_set_chunk_mb(int mb);       // spectral.cu

}  // namespace spgt

using namespace spgt;

extern "C" int spgt_set_tuning(const char* key, int value);

static int pick_cluster(int64_t BH, int S) {
    if (g_attn_cluster_override > 0) return g_attn_cluster_override;
    const int nsub = ceil_div(S, ATT_SUB);
    const int64_t slots = (int64_t)num_sms() * 2;
    int best = 1;
    int64_t best_cost = -1;
    for (int c = 1; c <= 8; c *= 2) {
        if (c > nsub) break;
        const int64_t waves = ceil_div(BH * c, slots);
        const int64_t per_warp = ceil_div((int64_t)ceil_div(nsub, c), (int64_t)ATT_WARPS);
        const int64_t cost = waves * (per_warp * 8 + 3);     // +3: fixed per-CTA reduction/sync overhead
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = c; }
    }
    return best;
}

template <int D>
static int launch_attn(const float* Q, const float* K, const float* V, float* out, float* t_out, int64_t BH, int H,
                       int S, int merged, cudaStream_t stream) {
    static SmemOptIn configured;
    auto kern = galerkin_attn_kernel<D>;
    if (int e = smem_opt_in(kern, AttnSmem<D>::BYTES, configured)) return e;
    const int C = pick_cluster(BH, S);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(BH * C), 1, 1);
    cfg.blockDim = dim3(ATT_THREADS, 1, 1);
    cfg.dynamicSmemBytes = AttnSmem<D>::BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, Q, K, V, out, t_out, S, H, merged);
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; (void)cudaGetLastError(); return SPGT_ERR_LAUNCH; }
    return launch_status();
}

extern "C" int spgt_galerkin_attn_fwd(const float* Q, const float* K, const float* V, float* out, float* t_out,
                                      int B, int H, int dpk, int S, int merged_heads, spgt_stream_t stream) {
    if (!Q || !K || !V || !out) return SPGT_ERR_NULL;
    if (B <= 0 || H <= 0 || S <= 0 || dpk < 32 || dpk > 35) return SPGT_ERR_SHAPE;
    const int64_t BH = (int64_t)B * H;
    if (BH * 8 > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(out)) return SPGT_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    if (g_attn_impl == 0) return launch_attn_tc(Q, K, V, out, t_out, BH, H, dpk, S, merged_heads, pick_cluster(BH, S), st);
    switch (dpk) {
        case 32: return launch_attn<32>(Q, K, V, out, t_out, BH, H, S, merged_heads, st);
        case 33: return launch_attn<33>(Q, K, V, out, t_out, BH, H, S, merged_heads, st);
        case 34: return launch_attn<34>(Q, K, V, out, t_out, BH, H, S, merged_heads, st);
        default: return launch_attn<35>(Q, K, V, out, t_out, BH, H, S, merged_heads, st);
    }
}

static int skinny_splits(int M, int N, int K, int batch) {
    const int64_t tiles = (int64_t)ceil_div(M, 32) * ceil_div(N, 32);
    const int nsub = ceil_div(K, 32);
    const int64_t slots = (int64_t)num_sms() * 4;
    int64_t s = ceil_div(slots, tiles * batch);
    const int64_t max_s = nsub >= 8 ? nsub / 8 : 1;     // at least two sub-tiles per warp
    if (s > max_s) s = max_s;
    if (s < 1) s = 1;
    if (s > 1024) s = 1024;
    return (int)s;
}

// Scratch of the two-pass kernels: one partial tile per (batch, tile, split).
static size_t skinny_twopass_bytes(int M, int N, int K, int batch) {
    const size_t tiles = (size_t)ceil_div(M, 32) * ceil_div(N, 32);
    return tiles * (size_t)batch * (size_t)skinny_splits(M, N, K, batch) * 1024 * sizeof(float);
}
// The one-launch kernel takes the shapes its 16-byte B chunks allow; its plan: P persistent CTAs over the k slices of all items.
static bool skinny_streamk_ok(int N) { return N % 4 == 0; }
static SksPlan skinny_plan(int M, int N, int K, int batch) {
    SksPlan pl;
    pl.tiles_n = ceil_div(N, 32); pl.tiles = ceil_div(M, 32) * pl.tiles_n; pl.nsub = ceil_div(K, SKS_K);
    pl.total = (int64_t)batch * pl.tiles * pl.nsub;
    const int64_t want = ceil_div(pl.total, (int64_t)(2 * SKS_WARPS));      // at least two slices per warp
    pl.P = (int)(want < num_sms() ? (want < 1 ? 1 : want) : num_sms());
    return pl;
}
// layout: pieces [2 P][1024] floats, then P tickets
static size_t skinny_streamk_bytes(const SksPlan& pl) { return (size_t)pl.P * (2 * 1024 * sizeof(float) + sizeof(unsigned int)); }

extern "C" size_t spgt_skinny_gemm_workspace_bytes(int M, int N, int K, int batch) {
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
    if (skinny_streamk_ok(N)) return skinny_streamk_bytes(skinny_plan(M, N, K, batch));
    return skinny_twopass_bytes(M, N, K, batch);
}

// Both entry points below run the same kernels on a scratch area: the one-launch kernel where the shape allows it,
// the two-pass kernels otherwise.  `scratch` holds at least spgt_skinny_gemm_workspace_bytes(M, N, K, batch) bytes.
static int skinny_launch(const float* A, const float* B, float* C, float alpha, int M, int N, int K, int batch, void* scratch,
                         cudaStream_t st) {
    if (skinny_streamk_ok(N)) {
        const SksPlan pl = skinny_plan(M, N, K, batch);
        static SmemOptIn configured;
        if (int e = smem_opt_in(skinny_streamk_kernel, SKS_SMEM, configured)) return e;
        float* pieces = (float*)scratch;
        unsigned int* tickets = (unsigned int*)(pieces + (size_t)pl.P * 2 * 1024);
        // The tickets count the finished pieces of an item and must start at zero.  The kernel leaves them at zero, but a
        // fresh workspace holds anything, so they are cleared on the stream before every launch (a few hundred bytes).
        if (cudaMemsetAsync(tickets, 0, (size_t)pl.P * sizeof(unsigned int), st) != cudaSuccess) return launch_status();
        skinny_streamk_kernel<<<pl.P, SKS_WARPS * 32, SKS_SMEM, st>>>(A, B, C, alpha, M, N, K, pl, pieces, tickets);
        return launch_status();
    }
    const int tiles_n = ceil_div(N, 32), tiles = ceil_div(M, 32) * tiles_n;
    const int splits = skinny_splits(M, N, K, batch);
    const int64_t blocks = (int64_t)tiles * splits * batch;
    if (blocks > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    const size_t smem = (size_t)SK_WARPS * SK_WARP_FLOATS * sizeof(float);
    if (int e = smem_opt_in(skinny_splitk_kernel, smem, g_skinny_smem)) return e;
    skinny_splitk_kernel<<<(unsigned)blocks, SK_WARPS * 32, smem, st>>>(A, B, (float*)scratch, M, N, K, tiles_n, tiles, splits, 0);
    if (int e = launch_status()) return e;
    skinny_reduce_kernel<<<(unsigned)((int64_t)tiles * batch), 256, 0, st>>>((const float*)scratch, C, alpha, M, N, tiles_n, tiles, splits);
    return launch_status();
}

extern "C" int spgt_batched_skinny_gemm(const float* A, const float* B, float* C, float alpha, int M, int N, int K,
                                        int batch, void* workspace, size_t workspace_bytes, spgt_stream_t stream) {
    if (!A || !B || !C) return SPGT_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return SPGT_ERR_SHAPE;
    if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return SPGT_ERR_ALIGN;
    const size_t need = spgt_skinny_gemm_workspace_bytes(M, N, K, batch);
    if (!workspace || workspace_bytes < need) return SPGT_ERR_WORKSPACE;
    if (!aligned16(workspace)) return SPGT_ERR_ALIGN;
    return skinny_launch(A, B, C, alpha, M, N, K, batch, workspace, (cudaStream_t)stream);
}

// ------------------------------------------------------------------------------------------------------------
// Batched skinny GEMM for callers that cannot hand over a workspace and must not allocate.
//
// Who needs this: a host that drives the library from inside a plugin callback, a real-time loop or a memory
// pool it does not own often has no way to obtain device memory at call time (its allocator may take a lock, may
// synchronise the device, or may simply be out of reach from the calling layer), and no place to keep a buffer
// between calls.  spgt_batched_skinny_gemm() asks such a caller for a workspace it cannot provide.  The entry
// point below runs the same kernels on the same plan - so its result is bit-identical - but takes the scratch
// (the partial tiles of the split k range and the tickets that count them) from a fixed array that is part of the
// loaded library image on every device.  It never calls cudaMalloc, cudaFree or any other allocating routine.
//
// Limit: the scratch must fit SPGT_SKINNY_NOALLOC_BYTES (8 MiB).  Larger problems are refused with
// SPGT_ERR_TOO_LARGE; nothing is launched in that case.  spgt_skinny_gemm_workspace_bytes() gives the size a
// problem needs, spgt_skinny_gemm_noalloc_max_bytes() the limit.
//
// Set-up: the first call on a device (with that device current) looks up the device address of the array once
// and caches it, and opts the kernels in to their shared-memory size.  Those are runtime queries - with lazy module
// loading that first call may also be what loads the module that holds the array - so make one call on every
// device you use before you start capturing a stream; later calls only clear the tickets and launch.
//
// Initial contents: every call shares the array and finds what the last call left.  The partial tiles need no
// clearing: each call writes every element of every tile it later reads.  The tickets must start at zero and are
// cleared on the stream (cudaMemsetAsync, no allocation) before each launch.
//
// Concurrency: there is one array per device.  Two calls whose kernels can overlap on the same device (different
// streams, or different host threads on different streams) would write the same partial tiles and race; issue
// the calls of one device on one stream, or order them with events.
// ------------------------------------------------------------------------------------------------------------
constexpr size_t SKINNY_NOALLOC_FLOATS = (size_t)2 * 1024 * 1024;                 // 8 MiB
static __device__ __align__(256) float g_skinny_noalloc_scratch[SKINNY_NOALLOC_FLOATS];

static float* g_skinny_noalloc_ptr[SPGT_MAX_DEVICES] = {};   // device address of the array, per device; 0 = not looked up

extern "C" size_t spgt_skinny_gemm_noalloc_max_bytes(void) { return SKINNY_NOALLOC_FLOATS * sizeof(float); }

extern "C" int spgt_batched_skinny_gemm_noalloc(const float* A, const float* B, float* C, float alpha, int M, int N,
                                                int K, int batch, spgt_stream_t stream) {
    if (!A || !B || !C) return SPGT_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return SPGT_ERR_SHAPE;
    if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return SPGT_ERR_ALIGN;
    if (spgt_skinny_gemm_workspace_bytes(M, N, K, batch) > SKINNY_NOALLOC_FLOATS * sizeof(float)) return SPGT_ERR_TOO_LARGE;

    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return launch_status();
    if (dev < 0 || dev >= SPGT_MAX_DEVICES) return SPGT_ERR_SHAPE;
    float* scratch = g_skinny_noalloc_ptr[dev];
    if (!scratch) {   // once per device: the address of this device's copy of the array
        cudaError_t e = cudaGetSymbolAddress((void**)&scratch, g_skinny_noalloc_scratch);
        if (e != cudaSuccess || !scratch) { g_last_cuda_error = (int)e; (void)cudaGetLastError(); return SPGT_ERR_LAUNCH; }
        g_skinny_noalloc_ptr[dev] = scratch;
    }
    return skinny_launch(A, B, C, alpha, M, N, K, batch, scratch, (cudaStream_t)stream);
}

extern "C" int spgt_set_tuning(const char* key, int value) {
    if (!key) return SPGT_ERR_NULL;
    auto eq = [&](const char* k) { int i = 0; while (k[i] && key[i] == k[i]) ++i; return k[i] == 0 && key[i] == 0; };
    if (eq("attn_cluster")) {
        if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8) return SPGT_ERR_SHAPE;
        g_attn_cluster_override = value;
        return SPGT_OK;
    }
    if (eq("spectral_chunk_mb")) {
        if (value < 0 || value > 65536) return SPGT_ERR_SHAPE;
        spectral_set_chunk_mb(value);
        return SPGT_OK;
    }
    if (eq("attn_impl")) {
        if (value != 0 && value != 1) return SPGT_ERR_SHAPE;
        g_attn_impl = value;
        return SPGT_OK;
    }
    return SPGT_ERR_SHAPE;
}
