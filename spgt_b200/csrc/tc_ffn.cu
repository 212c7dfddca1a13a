// Fused feed-forward block  y = act(x W1 + b1) W2 + b2 (+ residual)  for 128 -> 256 -> 128 on tcgen05 (3xTF32).
//
// The two GEMMs run back to back on one 128-row tile and the 128 x 256 hidden activations never leave the SM:
//   GEMM1  x rows (one per thread: hi / lo split, tcgen05.st) are the A operand in tensor memory, W1 streams through
//          shared memory as pre-split, pre-swizzled images (N = 256 per MMA: the MMA then occupies the pipe longer
//          than it takes to issue), accumulator D1 = 256 TMEM columns;
//   hidden the eight epilogue warps read D1 32 columns at a time, add b1, apply the activation, split and store the
//          result straight back into tensor memory as the A operand of GEMM2 (k-blocks of 32 hidden channels);
//   GEMM2  W2 streams like W1, accumulator D2 = 128 TMEM columns; its epilogue (bias, residual, coalesced stores through
//          a shared-memory staging slot) overlaps GEMM1 of the next tile.
// Tensor memory: D1 [0,256) | D2 [256,384) | two A stages of 64 columns (hi 32 | lo 32), used in turn by the 4 x
// k-blocks and the 8 hidden k-blocks of a tile.  Shared memory: a ring of four 32 KB weight slots (a W1 k-block takes
// two: hi and lo image of 256 rows; a W2 k-block one), a 3-stage raw ring for x, the epilogue staging.
// warps 0-3 x loaders, 4-7 x splitters, 8 weight loader, 9 MMA issuer, 10-17 hidden converters / epilogue.
// Every wait is a bounded mbarrier poll that records an error code on expiry (read back through spgt_tc_status).
#include "tc_common.cuh"

namespace spgt {

__device__ int g_ffn_status = 0;         // 0 = ok; otherwise the code (21..33) of the first wait that gave up

constexpr int FF_D = 128, FF_H = 256;
constexpr int FF_KB1 = FF_D / TC_BK, FF_KB2 = FF_H / TC_BK;          // 4 and 8 k-blocks
constexpr int FF_USES = FF_KB1 + FF_KB2;                             // A-stage uses per tile
constexpr int FF_WSLOT = 32768, FF_NW = 4;                           // weight ring
constexpr int FF_RAW = TC_BM * TC_BK * 4, FF_NR = 3;                 // raw x ring
constexpr int FF_SLOT_BYTES = 144, FF_EPI_WARPS = 8, FF_EPI_WARP0 = 10;
constexpr int FF_STAGING = 32 * FF_EPI_WARPS * FF_SLOT_BYTES;
constexpr int FF_THREADS = 32 * (FF_EPI_WARP0 + FF_EPI_WARPS);
constexpr int FF_CONST = (FF_H + FF_D) * 4;
constexpr size_t FF_SMEM = 1024 + (size_t)FF_NW * FF_WSLOT + FF_NR * FF_RAW + FF_STAGING + FF_CONST + 256;
constexpr uint32_t FF_D1 = 0, FF_D2 = 256, FF_A = 384;

__global__ void __launch_bounds__(FF_THREADS, 1)
tc_ffn_kernel(const float* __restrict__ x, int lda, const float* __restrict__ w1img, const float* __restrict__ b1,
              const float* __restrict__ w2img, const float* __restrict__ b2, const float* __restrict__ residual, int ldr,
              float* __restrict__ y, int ldc, int rows, int n_tiles_m, int act) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* raw = smem + FF_NW * FF_WSLOT;
    uint8_t* staging = raw + FF_NR * FF_RAW;
    float* consts = reinterpret_cast<float*>(staging + FF_STAGING);      // b1 [256] | b2 [128]
    uint8_t* bar_mem = staging + FF_STAGING + FF_CONST;
    const uint32_t bars = smem_u32(bar_mem);
    auto a_full = [&](int s) { return bars + 8u * s; };                 // [2] splitters / converters -> MMA
    auto a_empty = [&](int s) { return bars + 8u * (2 + s); };          // [2] MMA commit -> producers
    auto w_full = [&](int s) { return bars + 8u * (4 + s); };           // [4] bulk copies -> MMA
    auto w_empty = [&](int s) { return bars + 8u * (8 + s); };          // [4] MMA commit -> weight loader
    auto raw_full = [&](int s) { return bars + 8u * (12 + s); };        // [3] x loaders -> splitters
    auto raw_empty = [&](int s) { return bars + 8u * (15 + s); };       // [3] splitters -> x loaders
    const uint32_t d1_full = bars + 8u * 18, d1_empty = bars + 8u * 19, d2_full = bars + 8u * 20, d2_empty = bars + 8u * 21;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mem + 192);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 200);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < 2; ++s) { mbar_init(a_full(s), 128); mbar_init(a_empty(s), 1); }
        for (int s = 0; s < FF_NW; ++s) { mbar_init(w_full(s), 1); mbar_init(w_empty(s), 1); }
        for (int s = 0; s < FF_NR; ++s) { mbar_init(raw_full(s), 128); mbar_init(raw_empty(s), 128); }
        mbar_init(d1_full, 1); mbar_init(d1_empty, 32 * FF_EPI_WARPS);
        mbar_init(d2_full, 1); mbar_init(d2_empty, 32 * FF_EPI_WARPS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    for (int i = tid; i < FF_H + FF_D; i += FF_THREADS) consts[i] = i < FF_H ? __ldg(b1 + i) : (b2 != nullptr ? __ldg(b2 + i - FF_H) : 0.0f);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int n_my = ((int)blockIdx.x < n_tiles_m) ? (n_tiles_m - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (warp < 4) {
        // ------------------------------------------ x loaders ------------------------------------------
        uint32_t aoff[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) aoff[i] = tc_swz((tid >> 3) + 16 * i, tid & 7);
        const uint32_t raw_s = smem_u32(raw);
        uint32_t sr = 0, ph = 0;
        bool alive = true;
        for (int ti = 0; ti < n_my && alive; ++ti) {
            const int row0 = ((int)blockIdx.x + ti * (int)gridDim.x) * TC_BM + (tid >> 3);
            for (int kb = 0; kb < FF_KB1; ++kb) {
                if (!mbar_wait(raw_empty(sr), ph ^ 1, abort_flag, 21, &g_ffn_status)) { alive = false; break; }
                const uint32_t dst = raw_s + sr * FF_RAW;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int row = row0 + 16 * i;
                    const bool ok = row < rows;
                    const float* p = x + (int64_t)(ok ? row : 0) * lda + kb * TC_BK + (tid & 7) * 4;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + aoff[i]), "l"(p), "r"(ok ? 16 : 0) : "memory");
                }
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(raw_full(sr)) : "memory");
                if (++sr == FF_NR) { sr = 0; ph ^= 1u; }
            }
        }
        cp_async_wait_all();
    } else if (warp < 8) {
        // ------------------------------------------ x splitters ------------------------------------------
        const int q = warp & 3, r = q * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        uint32_t roff[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) roff[c] = tc_swz(r, c);
        uint32_t sr = 0, pr = 0;
        bool alive = true;
        for (int ti = 0; ti < n_my && alive; ++ti) {
            // The A stages are shared with the hidden k-blocks of the previous tile, which another group of warps
            // produces: a parity wait alone cannot tell "freed two uses ago" from "freed ten uses ago", so the splitters
            // first wait until GEMM2 of the previous tile has completed (every hidden stage has been consumed).
            if (ti > 0 && !mbar_wait(d2_full, (uint32_t)((ti - 1) & 1), abort_flag, 34, &g_ffn_status)) break;
            for (int kb = 0; kb < FF_KB1; ++kb) {
                const uint32_t use = (uint32_t)(ti * FF_USES + kb), sa = use & 1u, pa = (use >> 1) & 1u;
                if (!mbar_wait(raw_full(sr), pr, abort_flag, 22, &g_ffn_status)) { alive = false; break; }
                if (!mbar_wait(a_empty(sa), pa ^ 1, abort_flag, 23, &g_ffn_status)) { alive = false; break; }
                tc_fence_after();
                const uint8_t* src = raw + sr * FF_RAW;
                float4 v[8];
#pragma unroll
                for (int c = 0; c < 8; ++c) v[c] = *reinterpret_cast<const float4*>(src + roff[c]);
                const uint32_t a_hi = tmem_base + lane_addr + FF_A + sa * 64;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 w = v[4 * h + j];
                        split_tf32(w.x, hi[4 * j], lo[4 * j]); split_tf32(w.y, hi[4 * j + 1], lo[4 * j + 1]);
                        split_tf32(w.z, hi[4 * j + 2], lo[4 * j + 2]); split_tf32(w.w, hi[4 * j + 3], lo[4 * j + 3]);
                    }
                    tc_st16(a_hi + 16 * h, hi);
                    tc_st16(a_hi + 32 + 16 * h, lo);
                }
                mbar_arrive(raw_empty(sr));
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(a_full(sa));
                if (++sr == FF_NR) { sr = 0; pr ^= 1u; }
            }
        }
    } else if (warp == 8) {
        // ------------------------------------------ weight loader ------------------------------------------
        // W1 image of k-block kb: column tile nt (128 rows) at ((nt * 4 + kb) * 2 + {hi 0, lo 1}) * 16 KB;
        // W2 image of k-block kb: hi | lo contiguous, 32 KB, at kb * 32 KB.
        if (lane == 0) {
            uint32_t sw = 0, ph = 0;
            bool alive = true;
            auto take = [&]() { return mbar_wait(w_empty(sw), ph ^ 1, abort_flag, 24, &g_ffn_status); };
            auto adv = [&]() { if (++sw == FF_NW) { sw = 0; ph ^= 1u; } };
            for (int ti = 0; ti < n_my && alive; ++ti) {
                for (int kb = 0; kb < FF_KB1 && alive; ++kb)
                    for (int part = 0; part < 2 && alive; ++part) {          // hi slot, lo slot: 256 rows each
                        if (!take()) { alive = false; break; }
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(w_full(sw)), "r"(FF_WSLOT) : "memory");
                        for (int nt = 0; nt < 2; ++nt) {
                            const float* src = w1img + ((size_t)((nt * FF_KB1 + kb) * 2 + part)) * 4096;
                            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                         ::"r"(smem_base + sw * FF_WSLOT + nt * 16384), "l"(src), "r"(16384), "r"(w_full(sw)) : "memory");
                        }
                        adv();
                    }
                for (int kb = 0; kb < FF_KB2 && alive; ++kb) {
                    if (!take()) { alive = false; break; }
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(w_full(sw)), "r"(FF_WSLOT) : "memory");
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(smem_base + sw * FF_WSLOT), "l"(w2img + (size_t)kb * 8192), "r"(FF_WSLOT), "r"(w_full(sw)) : "memory");
                    adv();
                }
            }
        }
    } else if (warp == 9) {
        // ------------------------------------------ MMA issuer ------------------------------------------
        constexpr uint32_t idesc1 = tc_idesc(FF_H), idesc2 = tc_idesc(FF_D);
        uint32_t sw = 0, pw = 0;
        bool alive = true;
        auto wadv = [&]() { if (++sw == FF_NW) { sw = 0; pw ^= 1u; } };
        for (int ti = 0; ti < n_my && alive; ++ti) {
            const uint32_t tph = (uint32_t)(ti & 1);
            // GEMM1 into D1 (free once the converters have read the previous tile's hidden values)
            if (!mbar_wait(d1_empty, tph ^ 1, abort_flag, 25, &g_ffn_status)) break;
            tc_fence_after();
            for (int kb = 0; kb < FF_KB1 && alive; ++kb) {
                const uint32_t use = (uint32_t)(ti * FF_USES + kb), sa = use & 1u, pa = (use >> 1) & 1u;
                if (!mbar_wait(a_full(sa), pa, abort_flag, 26, &g_ffn_status)) { alive = false; break; }
                const uint32_t s_hi = sw, p_hi = pw; wadv();
                const uint32_t s_lo = sw, p_lo = pw; wadv();
                if (!mbar_wait(w_full(s_hi), p_hi, abort_flag, 27, &g_ffn_status)) { alive = false; break; }
                if (!mbar_wait(w_full(s_lo), p_lo, abort_flag, 27, &g_ffn_status)) { alive = false; break; }
                tc_fence_after();
                if (lane == 0) {
                    const uint64_t dbh = tc_smem_desc(smem_base + s_hi * FF_WSLOT), dbl = tc_smem_desc(smem_base + s_lo * FF_WSLOT);
                    const uint32_t ah0 = tmem_base + FF_A + sa * 64;
#pragma unroll
                    for (int k8 = 0; k8 < TC_BK / 8; ++k8) {
                        const uint64_t adv = (uint64_t)(k8 * 2);
                        const uint32_t ah = ah0 + k8 * 8, al = ah + 32;
                        tc_mma_tf32_ts(tmem_base + FF_D1, al, dbh + adv, idesc1, (kb > 0 || k8 > 0) ? 1u : 0u);
                        tc_mma_tf32_ts(tmem_base + FF_D1, ah, dbl + adv, idesc1, 1u);
                        tc_mma_tf32_ts(tmem_base + FF_D1, ah, dbh + adv, idesc1, 1u);
                    }
                    tc_commit(a_empty(sa));
                    tc_commit(w_empty(s_hi));
                    tc_commit(w_empty(s_lo));
                    if (kb == FF_KB1 - 1) tc_commit(d1_full);
                }
                __syncwarp();
            }
            if (!alive) break;
            // GEMM2 into D2 (free once the previous tile's epilogue has read it)
            if (!mbar_wait(d2_empty, tph ^ 1, abort_flag, 28, &g_ffn_status)) break;
            tc_fence_after();
            for (int kb = 0; kb < FF_KB2 && alive; ++kb) {
                const uint32_t use = (uint32_t)(ti * FF_USES + FF_KB1 + kb), sa = use & 1u, pa = (use >> 1) & 1u;
                if (!mbar_wait(a_full(sa), pa, abort_flag, 29, &g_ffn_status)) { alive = false; break; }
                const uint32_t s_w = sw, p_w = pw; wadv();
                if (!mbar_wait(w_full(s_w), p_w, abort_flag, 30, &g_ffn_status)) { alive = false; break; }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t b_hi = smem_base + s_w * FF_WSLOT;
                    const uint64_t dbh = tc_smem_desc(b_hi), dbl = tc_smem_desc(b_hi + FF_WSLOT / 2);
                    const uint32_t ah0 = tmem_base + FF_A + sa * 64;
#pragma unroll
                    for (int k8 = 0; k8 < TC_BK / 8; ++k8) {
                        const uint64_t adv = (uint64_t)(k8 * 2);
                        const uint32_t ah = ah0 + k8 * 8, al = ah + 32;
                        tc_mma_tf32_ts(tmem_base + FF_D2, al, dbh + adv, idesc2, (kb > 0 || k8 > 0) ? 1u : 0u);
                        tc_mma_tf32_ts(tmem_base + FF_D2, ah, dbl + adv, idesc2, 1u);
                        tc_mma_tf32_ts(tmem_base + FF_D2, ah, dbh + adv, idesc2, 1u);
                    }
                    tc_commit(a_empty(sa));
                    tc_commit(w_empty(s_w));
                    if (kb == FF_KB2 - 1) tc_commit(d2_full);
                }
                __syncwarp();
            }
        }
    } else {
        // ------------------------------------------ hidden converters + epilogue ------------------------------------------
        const int q = warp & 3, half = (warp - FF_EPI_WARP0) >> 2;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const int epi_idx = (warp - FF_EPI_WARP0) * 32 + lane;
        float* slot_ptr = reinterpret_cast<float*>(staging + epi_idx * FF_SLOT_BYTES);
        const uint8_t* warp_stage = staging + (warp - FF_EPI_WARP0) * 32 * FF_SLOT_BYTES;
        bool alive = true;
        for (int ti = 0; ti < n_my && alive; ++ti) {
            const uint32_t tph = (uint32_t)(ti & 1);
            // hidden k-blocks of this warp's parity: D1 -> bias, activation -> hi / lo -> A stage
            if (!mbar_wait(d1_full, tph, abort_flag, 31, &g_ffn_status)) break;
            tc_fence_after();
            for (int kb = half; kb < FF_KB2; kb += 2) {
                const uint32_t use = (uint32_t)(ti * FF_USES + FF_KB1 + kb), sa = use & 1u, pa = (use >> 1) & 1u;
                float v[32];
                tc_ld32(tmem_base + lane_addr + FF_D1 + kb * 32, v);
                if (kb + 2 >= FF_KB2) { tc_fence_before(); mbar_arrive(d1_empty); }          // last read of D1 by this thread
                uint32_t hi[32], lo[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) split_tf32(apply_act(v[j] + consts[kb * 32 + j], act), hi[j], lo[j]);
                if (!mbar_wait(a_empty(sa), pa ^ 1, abort_flag, 32, &g_ffn_status)) { alive = false; break; }
                tc_fence_after();
                const uint32_t a_hi = tmem_base + lane_addr + FF_A + sa * 64;
                tc_st16(a_hi, reinterpret_cast<uint32_t(&)[16]>(hi[0]));
                tc_st16(a_hi + 16, reinterpret_cast<uint32_t(&)[16]>(hi[16]));
                tc_st16(a_hi + 32, reinterpret_cast<uint32_t(&)[16]>(lo[0]));
                tc_st16(a_hi + 48, reinterpret_cast<uint32_t(&)[16]>(lo[16]));
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(a_full(sa));
            }
            if (!alive) break;
            // epilogue of GEMM2: columns [half * 64, +64) of the 128 outputs, 32 at a time through the staging slots.
            // The residual values of the elements this thread will store are fetched while GEMM2 is still running: a
            // load issued in the store phase queues behind the producers' traffic and stalls it for microseconds.
            const int tile = (int)blockIdx.x + ti * (int)gridDim.x;
            const int tile_row0 = tile * TC_BM + q * 32;
            float4 rres[8];
            auto res_fetch = [&](int c0_) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int orow = tile_row0 + i * 4 + (lane >> 3);
                    rres[i] = orow < rows ? __ldg(reinterpret_cast<const float4*>(residual + (int64_t)orow * ldr + c0_ + (lane & 7) * 4))
                                          : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            };
            if (residual != nullptr) res_fetch(half * 64);
            if (!mbar_wait(d2_full, tph, abort_flag, 33, &g_ffn_status)) break;
            tc_fence_after();
#pragma unroll
            for (int ps = 0; ps < 2; ++ps) {
                const int c0 = half * 64 + ps * 32;
#pragma unroll 1
                for (int cc = 0; cc < 32; cc += 16) {
                    float v[16];
                    tc_ld16(tmem_base + lane_addr + FF_D2 + c0 + cc, v);
#pragma unroll
                    for (int j4 = 0; j4 < 4; ++j4) {
                        const float4 b = *reinterpret_cast<const float4*>(consts + FF_H + c0 + cc + 4 * j4);
                        *reinterpret_cast<float4*>(slot_ptr + cc + 4 * j4) =
                            make_float4(v[4 * j4] + b.x, v[4 * j4 + 1] + b.y, v[4 * j4 + 2] + b.z, v[4 * j4 + 3] + b.w);
                    }
                }
                if (c0 + 32 >= half * 64 + 64) { tc_fence_before(); mbar_arrive(d2_empty); }   // D2 is in registers / staging
                __syncwarp();
                const int col = c0 + (lane & 7) * 4;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int rr = i * 4 + (lane >> 3);
                    const int orow = tile_row0 + rr;
                    if (orow < rows) {
                        float4 o = *reinterpret_cast<const float4*>(warp_stage + rr * FF_SLOT_BYTES + (lane & 7) * 16);
                        if (residual != nullptr) {
                            const float4 rv = rres[i];
                            o.x += rv.x; o.y += rv.y; o.z += rv.z; o.w += rv.w;
                        }
                        *reinterpret_cast<float4*>(y + (int64_t)orow * ldc + col) = o;
                    }
                }
                if (ps == 0 && residual != nullptr) res_fetch(half * 64 + 32);
                __syncwarp();
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

int ffn_tc_status_reset() {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_ffn_status, &zero, sizeof(int)) == cudaSuccess ? SPGT_OK : SPGT_ERR_LAUNCH;
}

int ffn_tc_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_ffn_status, sizeof(int)) != cudaSuccess) return SPGT_ERR_LAUNCH;
    return v;
}

}  // namespace spgt

using namespace spgt;

extern "C" int spgt_ffn_tc_fwd(const float* x, int lda, const void* w1prep, const float* b1, const void* w2prep, const float* b2,
                               const float* residual, int ldr, float* y, int ldc, int rows, int D, int Hd, int act,
                               spgt_stream_t stream) {
    if (!x || !w1prep || !b1 || !w2prep || !y) return SPGT_ERR_NULL;
    if (rows <= 0 || D != FF_D || Hd != FF_H || lda < D || ldc < D || (residual && ldr < D)) return SPGT_ERR_SHAPE;
    if ((lda & 3) || (ldc & 3) || (residual && (ldr & 3)) || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(w1prep) || !aligned16(w2prep) || !aligned16(y) || (residual && !aligned16(residual)) ||
        !aligned16(b1) || (b2 && !aligned16(b2)))
        return SPGT_ERR_ALIGN;
    static SmemOptIn configured;
    if (int e = smem_opt_in(tc_ffn_kernel, FF_SMEM, configured)) return e;
    const int n_tiles = ceil_div(rows, TC_BM);
    const int grid = n_tiles < num_sms() ? n_tiles : num_sms();
    tc_ffn_kernel<<<grid, FF_THREADS, FF_SMEM, (cudaStream_t)stream>>>(x, lda, (const float*)w1prep, b1, (const float*)w2prep, b2,
                                                                       residual, ldr, y, ldc, rows, n_tiles, act);
    return launch_status();
}
