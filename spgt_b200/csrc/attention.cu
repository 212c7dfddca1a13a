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

static SmemOptIn g_skinny_smem;           // shared-memory opt-in of skinny_splitk_kernel, per device
static int g_attn_cluster_override = 0;   // 0 = heuristic; set through spgt_set_tuning("attn_cluster", n)
static int g_attn_impl = 0;               // 0 = tcgen05 kernel (attention_tc.cu, default), 1 = warp-MMA kernel of this file

// defined in attention_tc.cu
int launch_attn_tc(const float* Q, const float* K, const float* V, float* out, float* t_out, int64_t BH, int H, int dpk,
                   int S, int merged, int cluster, cudaStream_t stream);

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

extern "C" size_t spgt_skinny_gemm_workspace_bytes(int M, int N, int K, int batch) {
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
    const size_t tiles = (size_t)ceil_div(M, 32) * ceil_div(N, 32);
    return tiles * (size_t)batch * (size_t)skinny_splits(M, N, K, batch) * 1024 * sizeof(float);
}

extern "C" int spgt_batched_skinny_gemm(const float* A, const float* B, float* C, float alpha, int M, int N, int K,
                                        int batch, void* workspace, size_t workspace_bytes, spgt_stream_t stream) {
    if (!A || !B || !C) return SPGT_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return SPGT_ERR_SHAPE;
    if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return SPGT_ERR_ALIGN;
    const size_t need = spgt_skinny_gemm_workspace_bytes(M, N, K, batch);
    if (!workspace || workspace_bytes < need) return SPGT_ERR_WORKSPACE;
    if (!aligned16(workspace)) return SPGT_ERR_ALIGN;
    const int tiles_n = ceil_div(N, 32), tiles = ceil_div(M, 32) * tiles_n;
    const int splits = skinny_splits(M, N, K, batch);
    const int64_t blocks = (int64_t)tiles * splits * batch;
    if (blocks > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    const size_t smem = (size_t)SK_WARPS * SK_WARP_FLOATS * sizeof(float);
    if (int e = smem_opt_in(skinny_splitk_kernel, smem, g_skinny_smem)) return e;
    cudaStream_t st = (cudaStream_t)stream;
    const int vecB = (N % 4 == 0) ? 1 : 0;
    skinny_splitk_kernel<<<(unsigned)blocks, SK_WARPS * 32, smem, st>>>(A, B, (float*)workspace, M, N, K, tiles_n, tiles,
                                                                     splits, vecB);
    if (int e = launch_status()) return e;
    skinny_reduce_kernel<<<(unsigned)((int64_t)tiles * batch), 256, 0, st>>>((const float*)workspace, C, alpha, M, N,
                                                                             tiles_n, tiles, splits);
    return launch_status();
}

// ------------------------------------------------------------------------------------------------------------
// Batched skinny GEMM for callers that cannot hand over a workspace and must not allocate.
//
// Who needs this: a host that drives the library from inside a plugin callback, a real-time loop or a memory
// pool it does not own often has no way to obtain device memory at call time (its allocator may take a lock, may
// synchronise the device, or may simply be out of reach from the calling layer), and no place to keep a buffer
// between calls.  spgt_batched_skinny_gemm() asks such a caller for a workspace it cannot provide.  The entry
// point below has the same arithmetic, but takes its split-K partial tiles from a fixed array that is part of
// the loaded library image on every device.  It never calls cudaMalloc, cudaFree or any other allocating routine.
//
// Limit: the partial tiles must fit SPGT_SKINNY_NOALLOC_BYTES (8 MiB).  Larger problems are refused with
// SPGT_ERR_TOO_LARGE; nothing is launched in that case.  spgt_skinny_gemm_workspace_bytes() gives the size a
// problem needs, spgt_skinny_gemm_noalloc_max_bytes() the limit.
//
// Set-up: the first call on a device (with that device current) looks up the device address of the array once
// and caches it.  That lookup is a runtime query, so make one call on every device you use before you start
// capturing a stream; later calls only launch the two kernels.
//
// Initial contents: nothing has to start at zero.  Pass 1 writes every element of every partial tile that pass 2
// reads, in the same call, so stale contents of an earlier call are never observed and no clearing kernel runs.
//
// Concurrency: there is one array per device.  Two calls whose kernels can overlap on the same device (different
// streams, or different host threads on different streams) would write the same partial tiles and race; issue
// the calls of one device on one stream, or order them with events.
// ------------------------------------------------------------------------------------------------------------
constexpr size_t SKINNY_NOALLOC_FLOATS = (size_t)2 * 1024 * 1024;                 // 8 MiB
static __device__ __align__(256) float g_skinny_noalloc_scratch[SKINNY_NOALLOC_FLOATS];

constexpr int SKINNY_MAX_DEVICES = 64;
static float* g_skinny_noalloc_ptr[SKINNY_MAX_DEVICES] = {};   // device address of the array, per device; 0 = not looked up

extern "C" size_t spgt_skinny_gemm_noalloc_max_bytes(void) { return SKINNY_NOALLOC_FLOATS * sizeof(float); }

extern "C" int spgt_batched_skinny_gemm_noalloc(const float* A, const float* B, float* C, float alpha, int M, int N,
                                                int K, int batch, spgt_stream_t stream) {
    if (!A || !B || !C) return SPGT_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return SPGT_ERR_SHAPE;
    if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return SPGT_ERR_ALIGN;
    const int tiles_n = ceil_div(N, 32), tiles = ceil_div(M, 32) * tiles_n;
    const int splits = skinny_splits(M, N, K, batch);
    const int64_t blocks = (int64_t)tiles * splits * batch;
    if (blocks > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    if ((size_t)blocks * 1024 > SKINNY_NOALLOC_FLOATS) return SPGT_ERR_TOO_LARGE;

    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return launch_status();
    if (dev < 0 || dev >= SKINNY_MAX_DEVICES) return SPGT_ERR_SHAPE;
    float* scratch = g_skinny_noalloc_ptr[dev];
    const size_t smem = (size_t)SK_WARPS * SK_WARP_FLOATS * sizeof(float);
    if (!scratch) {   // once per device: address of this device's copy of the array, and the kernel's shared-memory opt-in
        cudaError_t e = cudaGetSymbolAddress((void**)&scratch, g_skinny_noalloc_scratch);
        if (e != cudaSuccess || !scratch) { g_last_cuda_error = (int)e; (void)cudaGetLastError(); return SPGT_ERR_LAUNCH; }
        e = cudaFuncSetAttribute(skinny_splitk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) { g_last_cuda_error = (int)e; (void)cudaGetLastError(); return SPGT_ERR_LAUNCH; }
        g_skinny_noalloc_ptr[dev] = scratch;
    }
    cudaStream_t st = (cudaStream_t)stream;
    const int vecB = (N % 4 == 0) ? 1 : 0;
    skinny_splitk_kernel<<<(unsigned)blocks, SK_WARPS * 32, smem, st>>>(A, B, scratch, M, N, K, tiles_n, tiles, splits, vecB);
    if (int e = launch_status()) return e;
    skinny_reduce_kernel<<<(unsigned)((int64_t)tiles * batch), 256, 0, st>>>(scratch, C, alpha, M, N, tiles_n, tiles, splits);
    return launch_status();
}

extern "C" int spgt_set_tuning(const char* key, int value) {
    if (!key) return SPGT_ERR_NULL;
    auto eq = [&](const char* k) { int i = 0; while (k[i] && key[i] == k[i]) ++i; return k[i] == 0 && key[i] == 0; };
    if (eq("attn_cluster")) {
        if (value != 0 && value != 1 && value != 2 && value != 4 && value != 8) return SPGT_ERR_SHAPE;
        g_attn_cluster_override = value;
        return SPGT_OK;
    }
    if (eq("attn_impl")) {
        if (value != 0 && value != 1) return SPGT_ERR_SHAPE;
        g_attn_impl = value;
        return SPGT_OK;
    }
    return SPGT_ERR_SHAPE;
}
