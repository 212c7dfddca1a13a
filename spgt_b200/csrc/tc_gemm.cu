// Dense contractions on the 5th-generation tensor cores (tcgen05, accumulators in TMEM) with 3xTF32:
//   C[rows, N] = A[rows, K] * W[K, N],   A*W ~= A_lo*W_hi + A_hi*W_lo + A_hi*W_hi   (fp32-level accuracy).
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warps 0-3  loaders   : cp.async the raw fp32 A tile (dense rows or implicit-GEMM 3x3 gather) into 128B-swizzled
//                          K-major shared memory (completion tracked by an mbarrier); one thread bulk-copies the
//                          pre-split, pre-swizzled W_hi | W_lo image of the k-block;
//   warps 4-7  splitters : split the landed A tile in place into hi (tf32, round-to-nearest) and lo (x - hi);
//   warp  8    MMA       : one elected lane issues tcgen05.mma.kind::tf32 (128 x BN x 8) three times per k-step,
//                          tcgen05.commit releases the smem stage / publishes the accumulator;
//   warps 9-16 epilogue  : tcgen05.ld the 128 x BN fp32 accumulator (one row per thread, two warps per TMEM lane
//                          quarter splitting the columns) and run the fused epilogue while the MMA warp already
//                          works on the next tile (TMEM double buffer).
// All waits are bounded mbarrier polls: on expiry the kernel records an error code, stops waiting and returns.
#include "common.cuh"

namespace spgt {

constexpr int TC_BM = 128, TC_BK = 32;
constexpr int TC_PROD_THREADS = 128, TC_MMA_WARP = 8, TC_EPI_WARP0 = 9, TC_EPI_WARPS = 8, TC_THREADS = 32 * (9 + TC_EPI_WARPS);
constexpr uint32_t TC_SPIN_LIMIT = 1u << 24;

__device__ int g_tc_status = 0;          // 0 = ok; otherwise the code of the first wait that gave up

#ifdef SPGT_TC_TRACE                      // developer build only: per-tile timestamps of CTA 0 (see spgt_tc_trace_read)
__device__ long long g_tc_trace[64 * 16];
#define TC_TRACE(tile_i, slot) do { if (blockIdx.x == 0 && (tile_i) < 64) g_tc_trace[(tile_i) * 16 + (slot)] = clock64(); } while (0)
#else
#define TC_TRACE(tile_i, slot) do { } while (0)
#endif

// ---- mbarrier / tcgen05 primitives -------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded wait.  Returns false (and latches *abort_flag) when the limit is reached or another thread gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = code;
    atomicCAS(&g_tc_status, 0, code);
    return false;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], M = 128, N from the instruction descriptor, K = 8 (tf32)
__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t* u = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
        "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
          "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
          "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
          "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float* v) {
    uint32_t* u = reinterpret_cast<uint32_t*>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
          "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile with 128-byte rows, SWIZZLE_128B: 8-row groups are 1024 B apart (SBO), LBO unused (1),
// descriptor version 1 (sm_100), layout type 2.  The tile base must be 1024-byte aligned.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
__host__ __device__ constexpr uint32_t tc_idesc(int bn) {
    // c = f32 (1 << 4), a = b = tf32 (2 << 7, 2 << 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}
// byte offset of 16-byte chunk `c` (0..7) of row `r` inside a swizzled tile
__host__ __device__ __forceinline__ uint32_t tc_swz(int r, int c) { return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)); }

// ---- A-operand loaders (producer side; 128 threads, thread -> chunk (t & 7) of rows (t >> 3) + 16 i) ---------
struct TcDense {
    const float* x; int lda; int rows; int K;
    const float* rp[8]; bool rok[8]; int kc; bool kok;
    __device__ void init(int row0, int t) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int row = row0 + (t >> 3) + 16 * i;
            rok[i] = row < rows;
            rp[i] = x + (int64_t)(rok[i] ? row : 0) * lda;
        }
    }
    __device__ void set_k(int k0, int t) { kc = k0 + (t & 7) * 4; kok = kc < K; if (!kok) kc = 0; }
    __device__ const float* ptr(int i, bool& ok) const { ok = rok[i] && kok; return rp[i] + kc; }
};
struct TcConv {          // 3x3, padding 1, NHWC; K = 9 * Cin with Cin % 4 == 0
    const float* x; int cin_pitch, cin_off, Cin, Hh, Ww; int rows; int K;
    const float* rp[8]; int py[8], px[8]; int dy, dx, coff; bool kok;
    __device__ void init(int row0, int t) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int row = row0 + (t >> 3) + 16 * i;
            if (row < rows) {
                const int b = row / (Hh * Ww);
                const int rem = row - b * Hh * Ww;
                py[i] = rem / Ww; px[i] = rem - py[i] * Ww;
                rp[i] = x + (int64_t)row * cin_pitch + cin_off;
            } else { py[i] = -(1 << 20); px[i] = 0; rp[i] = x; }
        }
    }
    __device__ void set_k(int k0, int t) {
        const int k = k0 + (t & 7) * 4;
        kok = k < K;
        const int tap = kok ? k / Cin : 4;
        const int c = kok ? k - tap * Cin : 0;
        dy = tap / 3 - 1; dx = tap % 3 - 1;
        coff = (dy * Ww + dx) * cin_pitch + c;
    }
    __device__ const float* ptr(int i, bool& ok) const {
        const int yy = py[i] + dy, xx = px[i] + dx;
        ok = kok && yy >= 0 && yy < Hh && xx >= 0 && xx < Ww;
        return ok ? rp[i] + coff : x;
    }
};

// ---- epilogues (epilogue side; thread = one row of the 128-row tile, columns arrive 32 at a time) -----------
struct TcLinearEpi {
    const float* bias; const float* residual; int ldr; float* y; int ldc; int N; int act;
};
struct TcProjEpi {          // column tile p = 0,1,2 -> q, k, v; 128 columns = 4 heads of 32
    const float* bias[3]; const float* lnw[3]; const float* lnb[3]; float* out[3]; const float* pos;
    float eps; int S, H, d_pos;
};
struct TcHeadEpi {
    const float* b1; const float* w2; float b2, scale, shift; const float* scale_map; const float* shift_map;
    int dirichlet, Hh, Ww, act; float* out;
};

template <int BN> struct TcSmem {
    static constexpr int A_BYTES = TC_BM * TC_BK * 4;           // 16 KB
    static constexpr int B_BYTES = BN * TC_BK * 4;
    static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;     // A_hi(raw), A_lo, B_hi, B_lo
    static constexpr int STAGES = (BN > 64) ? 3 : 4;
    static constexpr int STAGING_BYTES = (2 * 128 + 256) * 4;         // partial row sums of epilogue warp pairs + b1 | w2 of the head
    static constexpr int BAR_BYTES = 192;
    static constexpr size_t BYTES = 1024 /*alignment slack*/ + (size_t)STAGES * STAGE_BYTES + STAGING_BYTES + BAR_BYTES;
};

enum { EPI_LINEAR = 0, EPI_PROJ = 1, EPI_HEAD = 2 };

template <int BN, class Loader, int EPI, class EpiParams>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_gemm_kernel(Loader ld, const float* __restrict__ wimg, int kpad, int rows, int n_tiles, int m_tiles, EpiParams ep) {
    using L = TcSmem<BN>;
    constexpr int ST = L::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;          // 1024-aligned for the 128B swizzle
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t stage0 = smem_base;
    const uint32_t bars = smem_base + ST * L::STAGE_BYTES + L::STAGING_BYTES;
    // barrier slots (8 bytes each): full[4], empty[4], raw[4], acc_full[2], acc_empty[2]; then tmem ptr, abort flag
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (4 + s); };
    auto raw_bar = [&](int s) { return bars + 8u * (8 + s); };
    auto accf_bar = [&](int b) { return bars + 8u * (12 + b); };
    auto acce_bar = [&](int b) { return bars + 8u * (14 + b); };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + ST * L::STAGE_BYTES + L::STAGING_BYTES + 128);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + ST * L::STAGE_BYTES + L::STAGING_BYTES + 144);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr int TMEM_COLS = (2 * BN <= 64) ? 64 : (2 * BN <= 128 ? 128 : 256);

    if (tid == 0) {
        for (int s = 0; s < ST; ++s) { mbar_init(full_bar(s), TC_PROD_THREADS + 1); mbar_init(empty_bar(s), 1); mbar_init(raw_bar(s), TC_PROD_THREADS); }
        for (int b = 0; b < 2; ++b) { mbar_init(accf_bar(b), 1); mbar_init(acce_bar(b), 32 * TC_EPI_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if constexpr (EPI == EPI_HEAD) {
        float* cst = reinterpret_cast<float*>(smem + ST * L::STAGE_BYTES) + 256;
        for (int i = tid; i < 256; i += TC_THREADS) cst[i] = i < 128 ? __ldg(ep.b1 + i) : __ldg(ep.w2 + i - 128);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int KB = kpad / TC_BK;
    const int total_tiles = m_tiles * n_tiles;

    if (warp < 4) {
        // ------------------------------------------ loaders ------------------------------------------
        const int t = tid;
        uint32_t it = 0;
        uint32_t aoff[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) aoff[i] = tc_swz((t >> 3) + 16 * i, t & 7);
        bool alive = true;
        for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x) {
            const int row0 = (tile / n_tiles) * TC_BM;
            ld.init(row0, t);
            if (t == 0) TC_TRACE(it / KB, 0);
            const float* wtile = wimg + (int64_t)(tile % n_tiles) * KB * (2 * L::B_BYTES / 4);
            for (int kb = 0; kb < KB; ++kb, ++it) {
                const uint32_t s = it % ST, ph = (it / ST) & 1;
                if (!mbar_wait(empty_bar(s), ph ^ 1, abort_flag, 1)) { alive = false; break; }
                const uint32_t a_hi = stage0 + s * L::STAGE_BYTES;
                if (t == 0) {      // the pre-swizzled W_hi | W_lo image of this (column tile, k-block): one bulk copy
                    const uint32_t bytes = 2 * L::B_BYTES;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full_bar(s)), "r"(bytes) : "memory");
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(a_hi + 2 * L::A_BYTES), "l"(wtile + (int64_t)kb * (2 * L::B_BYTES / 4)), "r"(bytes), "r"(full_bar(s)) : "memory");
                }
                ld.set_k(kb * TC_BK, t);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    bool ok;
                    const float* p = ld.ptr(i, ok);
                    const int n = ok ? 16 : 0;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(a_hi + aoff[i]), "l"(p), "r"(n) : "memory");
                }
                // arrive on raw[s] once every cp.async issued so far by this thread has landed
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(raw_bar(s)) : "memory");
            }
            if (t == 0) TC_TRACE((it - 1) / KB, 1);
        }
        cp_async_wait_all();
    } else if (warp < 8) {
        // ------------------------------------------ splitters ------------------------------------------
        const int t = tid - 128;
        uint32_t it = 0;
        uint32_t aoff[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) aoff[i] = tc_swz((t >> 3) + 16 * i, t & 7);
        bool alive = true;
        for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x) {
            for (int kb = 0; kb < KB; ++kb, ++it) {
                const uint32_t s = it % ST, ph = (it / ST) & 1;
                if (!mbar_wait(raw_bar(s), ph, abort_flag, 5)) { alive = false; break; }
                if (t == 0 && kb == 0) TC_TRACE(it / KB, 2);
                uint8_t* a_hi = smem + s * L::STAGE_BYTES;
                uint8_t* a_lo = a_hi + L::A_BYTES;
                float4 v[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = *reinterpret_cast<float4*>(a_hi + aoff[i]);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    uint32_t h[4], l[4];
                    split_tf32(v[i].x, h[0], l[0]); split_tf32(v[i].y, h[1], l[1]);
                    split_tf32(v[i].z, h[2], l[2]); split_tf32(v[i].w, h[3], l[3]);
                    *reinterpret_cast<uint4*>(a_hi + aoff[i]) = make_uint4(h[0], h[1], h[2], h[3]);
                    *reinterpret_cast<uint4*>(a_lo + aoff[i]) = make_uint4(l[0], l[1], l[2], l[3]);
                }
                fence_proxy_async();                     // generic-proxy writes -> visible to the tensor core
                mbar_arrive(full_bar(s));
                if (t == 0 && kb == KB - 1) TC_TRACE(it / KB, 3);
            }
        }
    } else if (warp == TC_MMA_WARP) {
        // ------------------------------------------ MMA issuer ------------------------------------------
        constexpr uint32_t idesc = tc_idesc(BN);
        uint32_t it = 0, ti = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x, ++ti) {
            const uint32_t buf = ti & 1, aph = (ti >> 1) & 1;
            if (lane == 0) TC_TRACE(ti, 4);
            if (!mbar_wait(acce_bar(buf), aph ^ 1, abort_flag, 2)) { alive = false; break; }
            if (lane == 0) TC_TRACE(ti, 5);
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * BN;
            for (int kb = 0; kb < KB; ++kb, ++it) {
                const uint32_t s = it % ST, ph = (it / ST) & 1;
                if (!mbar_wait(full_bar(s), ph, abort_flag, 3)) { alive = false; break; }
                if (lane == 0 && kb == 0) TC_TRACE(ti, 6);
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t a_hi = stage0 + s * L::STAGE_BYTES;
                    const uint64_t dah = tc_smem_desc(a_hi), dal = tc_smem_desc(a_hi + L::A_BYTES);
                    const uint64_t dbh = tc_smem_desc(a_hi + 2 * L::A_BYTES), dbl = tc_smem_desc(a_hi + 2 * L::A_BYTES + L::B_BYTES);
#pragma unroll
                    for (int k8 = 0; k8 < TC_BK / 8; ++k8) {
                        const uint64_t adv = (uint64_t)(k8 * 2);          // 32 bytes per k-step, in 16-byte units
                        tc_mma_tf32(d_tmem, dal + adv, dbh + adv, idesc, (kb > 0 || k8 > 0) ? 1u : 0u);
                        tc_mma_tf32(d_tmem, dah + adv, dbl + adv, idesc, 1u);
                        tc_mma_tf32(d_tmem, dah + adv, dbh + adv, idesc, 1u);
                    }
                    tc_commit(empty_bar(s));           // stage reusable once these MMAs have read it
                }
                __syncwarp();
            }
            if (alive && lane == 0) tc_commit(accf_bar(buf));
            if (lane == 0) TC_TRACE(ti, 7);
            __syncwarp();
        }
    } else {
        // ------------------------------------------ epilogue ------------------------------------------
        const int q = warp & 3;                        // TMEM lane quarter this warp may access
        const int half = (warp - TC_EPI_WARP0) >> 2;   // which half of the column chunks this warp of the pair takes
        const int r_in_tile = q * 32 + lane;
        uint32_t ti = 0;
        bool alive = true;
        for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x, ++ti) {
            const uint32_t buf = ti & 1, aph = (ti >> 1) & 1;
            if (tid == TC_EPI_WARP0 * 32) TC_TRACE(ti, 8);
            if (!mbar_wait(accf_bar(buf), aph, abort_flag, 4)) { alive = false; break; }
            if (tid == TC_EPI_WARP0 * 32) TC_TRACE(ti, 9);
            tc_fence_after();
            const int mt = tile / n_tiles, nt = tile % n_tiles;
            const int row = mt * TC_BM + r_in_tile;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN;

            if constexpr (EPI == EPI_LINEAR) {
                const TcLinearEpi& e = ep;
                const bool vec = ((e.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(e.y) & 15) == 0) &&
                                 (e.residual == nullptr || (((e.ldr & 3) == 0) && ((reinterpret_cast<uintptr_t>(e.residual) & 15) == 0)));
                constexpr int NCH = (BN + 31) / 32;
#pragma unroll 1
                for (int ch = half; ch < NCH; ch += 2) {
                    const int c0 = ch * 32;
                    float v[32];
                    if (BN - c0 >= 32) { tc_ld32(taddr + c0, v); }
                    else { tc_ld16(taddr + c0, v);
#pragma unroll
                        for (int j = 16; j < 32; ++j) v[j] = 0.0f; }
                    if (tid == TC_EPI_WARP0 * 32) TC_TRACE(ti, 11 + (ch >> 1) * 2);
                    if (row < rows) {
                        const int colb = nt * BN + c0;
                        float* yp = e.y + (int64_t)row * e.ldc + colb;
                        const float* rp = e.residual ? e.residual + (int64_t)row * e.ldr + colb : nullptr;
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const int col = colb + 4 * j4;
                            if (c0 + 4 * j4 >= BN || col >= e.N) continue;
                            if (vec && col + 3 < e.N) {
                                float4 b = e.bias ? __ldg(reinterpret_cast<const float4*>(e.bias + col)) : make_float4(0, 0, 0, 0);
                                float4 o;
                                o.x = apply_act(v[4 * j4] + b.x, e.act); o.y = apply_act(v[4 * j4 + 1] + b.y, e.act);
                                o.z = apply_act(v[4 * j4 + 2] + b.z, e.act); o.w = apply_act(v[4 * j4 + 3] + b.w, e.act);
                                if (rp) {
                                    const float4 r = __ldg(reinterpret_cast<const float4*>(rp + 4 * j4));
                                    o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
                                }
                                *reinterpret_cast<float4*>(yp + 4 * j4) = o;
                            } else {
#pragma unroll
                                for (int k = 0; k < 4; ++k) {
                                    if (col + k < e.N) {
                                        float o = apply_act(v[4 * j4 + k] + (e.bias ? __ldg(e.bias + col + k) : 0.0f), e.act);
                                        if (rp) o += __ldg(rp + 4 * j4 + k);
                                        yp[4 * j4 + k] = o;
                                    }
                                }
                            }
                        }
                    }
                    if (tid == TC_EPI_WARP0 * 32) TC_TRACE(ti, 12 + (ch >> 1) * 2);
                }
            } else if constexpr (EPI == EPI_PROJ) {
                const TcProjEpi& e = ep;
                const int p = nt;                               // 0: q, 1: k, 2: v
                const int dpk = e.d_pos + 32;
                const bool rok = row < rows;
                const int b = rok ? row / e.S : 0, s_ = rok ? row - b * e.S : 0;
                float* out = e.out[p];
                const float* bias = e.bias[p];
                const float* lnw = e.lnw[p];
                const float* lnb = e.lnb[p];
#pragma unroll 1
                for (int hd = half; hd < 4; hd += 2) {           // one head = 32 columns = one TMEM load
                    float v[32];
                    tc_ld32(taddr + hd * 32, v);
                    if (bias) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] += __ldg(bias + hd * 32 + j);
                    }
                    if (lnw != nullptr) {
                        float s = 0.0f;
#pragma unroll
                        for (int j = 0; j < 32; ++j) s += v[j];
                        const float mu = s * (1.0f / 32.0f);
                        float qq = 0.0f;
#pragma unroll
                        for (int j = 0; j < 32; ++j) { const float d = v[j] - mu; qq += d * d; }
                        const float inv = 1.0f / sqrtf(qq * (1.0f / 32.0f) + e.eps);
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            v[j] = (v[j] - mu) * inv * __ldg(lnw + hd * 32 + j) + __ldg(lnb + hd * 32 + j);
                    }
                    if (rok) {
                        float* o = out + (((int64_t)b * e.H + hd) * dpk + e.d_pos) * e.S + s_;
#pragma unroll
                        for (int j = 0; j < 32; ++j) o[(int64_t)j * e.S] = v[j];     // lanes = consecutive s: coalesced
                        for (int pp = 0; pp < e.d_pos; ++pp)
                            out[(((int64_t)b * e.H + hd) * dpk + pp) * e.S + s_] = __ldg(e.pos + (int64_t)row * e.d_pos + pp);
                    }
                }
            } else {
                const TcHeadEpi& e = ep;
                float* part = reinterpret_cast<float*>(smem + ST * L::STAGE_BYTES);   // [2][128] partial row sums
                const float4* cb = reinterpret_cast<const float4*>(part + 256);              // b1[128] then w2[128]
                float acc = 0.0f;
#pragma unroll 1
                for (int ch = half; ch < BN / 32; ch += 2) {
                    const int c0 = ch * 32;
                    float v[32];
                    tc_ld32(taddr + c0, v);
                    auto dot = [&](auto actf) {
#pragma unroll
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const float4 b = cb[(c0 >> 2) + j4], w = cb[32 + (c0 >> 2) + j4];
                            acc = fmaf(actf(v[4 * j4] + b.x), w.x, acc);
                            acc = fmaf(actf(v[4 * j4 + 1] + b.y), w.y, acc);
                            acc = fmaf(actf(v[4 * j4 + 2] + b.z), w.z, acc);
                            acc = fmaf(actf(v[4 * j4 + 3] + b.w), w.w, acc);
                        }
                    };
                    if (e.act == SPGT_ACT_SILU) dot([](float x) { return silu_f(x); });
                    else if (e.act == SPGT_ACT_RELU) dot([](float x) { return fmaxf(x, 0.0f); });
                    else if (e.act == SPGT_ACT_SILU2) dot([](float x) { return silu_f(silu_f(x)); });
                    else dot([](float x) { return x; });
                }
                if (half == 1) part[(ti & 1) * 128 + r_in_tile] = acc;
                asm volatile("bar.sync 1, %0;" ::"n"(32 * TC_EPI_WARPS) : "memory");   // epilogue warps only
                if (half == 0 && row < rows) {
                    acc += part[(ti & 1) * 128 + r_in_tile];
                    const int rem = row % (e.Hh * e.Ww);
                    const float sc = e.scale_map ? __ldg(e.scale_map + rem) : e.scale;
                    const float sh = e.shift_map ? __ldg(e.shift_map + rem) : e.shift;
                    float o = (acc + e.b2) * sc + sh;
                    if (e.dirichlet) {
                        const int y = rem / e.Ww, x = rem - y * e.Ww;
                        if (y == 0 || x == 0 || y == e.Hh - 1 || x == e.Ww - 1) o = 0.0f;
                    }
                    e.out[row] = o;
                }
            }
            tc_fence_before();
            mbar_arrive(acce_bar(buf));
            if (tid == TC_EPI_WARP0 * 32) TC_TRACE(ti, 10);
        }
    }
    // teardown: everyone meets, then the allocating warp frees the tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == TC_MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- weight preparation: [K][ldw] row-major fp32 -> per (column tile, k-block) the exact shared-memory image the
// kernel needs: W_hi then W_lo, each [bn rows (n)][32 k] K-major with the 128-byte swizzle applied, zero padded.
__global__ void tc_weight_prepare_kernel(const float* __restrict__ w, int ldw, int K, int N, int kpad, int npad, int bn,
                                         float* __restrict__ img) {
    const int64_t total = (int64_t)npad * kpad;
    const int KB = kpad / TC_BK;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int n = (int)(i / kpad), k = (int)(i % kpad);
        const float v = (n < N && k < K) ? __ldg(w + (int64_t)k * ldw + n) : 0.0f;
        uint32_t h, l;
        split_tf32(v, h, l);
        uint32_t l2;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l2) : "f"(__uint_as_float(l)));
        const int nt = n / bn, r = n % bn, kb = k / TC_BK, kk = k % TC_BK;
        const int64_t blk = ((int64_t)nt * KB + kb) * (2 * bn * TC_BK);
        const int off = (int)(tc_swz(r, kk >> 2) >> 2) + (kk & 3);
        img[blk + off] = __uint_as_float(h);
        img[blk + bn * TC_BK + off] = __uint_as_float(l2);
    }
}

static int tc_bn_for(int N) { return N <= 32 ? 32 : (N <= 48 ? 48 : (N <= 64 ? 64 : 128)); }

template <int BN, class Loader, int EPI, class EpiParams>
static int tc_launch(Loader ld, const float* wimg, int kpad, int rows, int n_tiles, const EpiParams& ep, cudaStream_t st) {
    static bool done = false;
    auto kern = tc_gemm_kernel<BN, Loader, EPI, EpiParams>;
    if (!done) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcSmem<BN>::BYTES) != cudaSuccess) return launch_status();
        done = true;
    }
    const int m_tiles = ceil_div(rows, TC_BM);
    const int64_t tiles = (int64_t)m_tiles * n_tiles;
    const int grid = (int)(tiles < num_sms() ? tiles : num_sms());
    kern<<<grid, TC_THREADS, TcSmem<BN>::BYTES, st>>>(ld, wimg, kpad, rows, n_tiles, m_tiles, ep);
    return launch_status();
}

template <class Loader>
static int tc_dispatch_linear(Loader ld, const float* wprep, int K, int N, int rows, const TcLinearEpi& ep, cudaStream_t st) {
    const int bn = tc_bn_for(N), kpad = ceil_div(K, TC_BK) * TC_BK, npad = ceil_div(N, bn) * bn;
    const int n_tiles = npad / bn;
    switch (bn) {
        case 32: return tc_launch<32, Loader, EPI_LINEAR, TcLinearEpi>(ld, wprep, kpad, rows, n_tiles, ep, st);
        case 48: return tc_launch<48, Loader, EPI_LINEAR, TcLinearEpi>(ld, wprep, kpad, rows, n_tiles, ep, st);
        case 64: return tc_launch<64, Loader, EPI_LINEAR, TcLinearEpi>(ld, wprep, kpad, rows, n_tiles, ep, st);
        default: return tc_launch<128, Loader, EPI_LINEAR, TcLinearEpi>(ld, wprep, kpad, rows, n_tiles, ep, st);
    }
}

}  // namespace spgt

using namespace spgt;

extern "C" size_t spgt_tc_weight_bytes(int K, int N) {
    if (K <= 0 || N <= 0) return 0;
    const int bn = tc_bn_for(N);
    return (size_t)2 * (ceil_div(N, bn) * bn) * (ceil_div(K, TC_BK) * TC_BK) * sizeof(float);
}

extern "C" int spgt_tc_weight_prepare(const float* w_kn, int ldw, int K, int N, void* out, size_t out_bytes,
                                      spgt_stream_t stream) {
    if (!w_kn || !out) return SPGT_ERR_NULL;
    if (K <= 0 || N <= 0 || ldw < N) return SPGT_ERR_SHAPE;
    if (out_bytes < spgt_tc_weight_bytes(K, N)) return SPGT_ERR_WORKSPACE;
    if (!aligned16(out)) return SPGT_ERR_ALIGN;
    const int bn = tc_bn_for(N), kpad = ceil_div(K, TC_BK) * TC_BK, npad = ceil_div(N, bn) * bn;
    tc_weight_prepare_kernel<<<ceil_div(npad * kpad, 256), 256, 0, (cudaStream_t)stream>>>(w_kn, ldw, K, N, kpad, npad, bn,
                                                                                         (float*)out);
    return launch_status();
}

#ifdef SPGT_TC_TRACE
extern "C" int spgt_tc_trace_read(long long* host_out) {   // 64 tiles x 16 slots of clock64() values of CTA 0
    return cudaMemcpyFromSymbol(host_out, g_tc_trace, sizeof(long long) * 64 * 16) == cudaSuccess ? 0 : SPGT_ERR_LAUNCH;
}
#endif

extern "C" int spgt_tc_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return SPGT_ERR_LAUNCH;
    return v;
}

extern "C" int spgt_linear_tc_fwd(const float* x, int lda, const void* wprep, const float* bias, const float* residual,
                                  int ldr, float* y, int ldc, int rows, int K, int N, int act, spgt_stream_t stream) {
    if (!x || !wprep || !y) return SPGT_ERR_NULL;
    if (rows <= 0 || K <= 0 || N <= 0 || lda < K || ldc < N || (residual && ldr < N)) return SPGT_ERR_SHAPE;
    if ((lda & 3) || (K & 3) || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(wprep) || !aligned16(y)) return SPGT_ERR_ALIGN;
    TcDense ld;
    ld.x = x; ld.lda = lda; ld.rows = rows; ld.K = K;
    TcLinearEpi ep{bias, residual, ldr, y, ldc, N, act};
    return tc_dispatch_linear(ld, (const float*)wprep, K, N, rows, ep, (cudaStream_t)stream);
}

extern "C" int spgt_conv3x3_tc_fwd(const float* x, int cin_pitch, int cin_off, int Cin, const void* wprep, const float* bias,
                                   float* y, int cout_pitch, int cout_off, int Cout, int B, int Hh, int Ww, int act,
                                   spgt_stream_t stream) {
    if (!x || !wprep || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hh <= 0 || Ww <= 0 || Cin <= 0 || Cout <= 0 || cin_off < 0 || cout_off < 0) return SPGT_ERR_SHAPE;
    if (cin_off + Cin > cin_pitch || cout_off + Cout > cout_pitch || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if ((Cin & 3) || (cin_off & 3) || (cin_pitch & 3)) return SPGT_ERR_SHAPE;
    const int64_t rows64 = (int64_t)B * Hh * Ww;
    if (rows64 > 0x7fffffffLL / 4 || rows64 * cin_pitch > 0x7fffffffLL * 4) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(wprep) || !aligned16(y)) return SPGT_ERR_ALIGN;
    TcConv ld;
    ld.x = x; ld.cin_pitch = cin_pitch; ld.cin_off = cin_off; ld.Cin = Cin; ld.Hh = Hh; ld.Ww = Ww; ld.rows = (int)rows64; ld.K = 9 * Cin;
    TcLinearEpi ep{bias, nullptr, 0, y + cout_off, cout_pitch, Cout, act};
    return tc_dispatch_linear(ld, (const float*)wprep, 9 * Cin, Cout, (int)rows64, ep, (cudaStream_t)stream);
}

extern "C" int spgt_projpos_qkv_tc_fwd(const float* x, const void* wprep_qkv, const float* bq, const float* bk, const float* bv,
                                       const float* lnwk, const float* lnbk, const float* lnwv, const float* lnbv, float eps,
                                       const float* pos, float* q, float* k, float* v, int B, int S, int D, int H, int d_head,
                                       int d_pos, spgt_stream_t stream) {
    if (!x || !wprep_qkv || !q || !k || !v || !lnwk || !lnbk || !lnwv || !lnbv) return SPGT_ERR_NULL;
    if (B <= 0 || S <= 0 || D != 128 || H != 4 || d_head != 32 || d_pos < 0 || d_pos > 8) return SPGT_ERR_SHAPE;
    if (d_pos > 0 && !pos) return SPGT_ERR_NULL;
    const int64_t rows64 = (int64_t)B * S;
    if (rows64 > 0x7fffffffLL / 2) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(wprep_qkv) || !aligned16(q) || !aligned16(k) || !aligned16(v)) return SPGT_ERR_ALIGN;
    TcDense ld;
    ld.x = x; ld.lda = D; ld.rows = (int)rows64; ld.K = D;
    TcProjEpi ep = {};
    ep.bias[0] = bq; ep.bias[1] = bk; ep.bias[2] = bv;
    ep.lnw[1] = lnwk; ep.lnb[1] = lnbk; ep.lnw[2] = lnwv; ep.lnb[2] = lnbv;
    ep.out[0] = q; ep.out[1] = k; ep.out[2] = v; ep.pos = pos; ep.eps = eps; ep.S = S; ep.H = H; ep.d_pos = d_pos;
    // wprep_qkv is prepared from the [128, 384] concatenation of Wq | Wk | Wv: three column tiles of 128
    return tc_launch<128, TcDense, EPI_PROJ, TcProjEpi>(ld, (const float*)wprep_qkv, 128, (int)rows64, 3, ep, (cudaStream_t)stream);
}

extern "C" int spgt_decoder_head_tc_fwd(const float* x, const void* w1prep, const float* b1, const float* w2, float b2,
                                        float scale, float shift, const float* scale_map, const float* shift_map,
                                        int dirichlet, float* out, int B, int Hh, int Ww, int K, int N1, int act,
                                        spgt_stream_t stream) {
    if (!x || !w1prep || !b1 || !w2 || !out) return SPGT_ERR_NULL;
    if (B <= 0 || Hh <= 0 || Ww <= 0 || K <= 0 || (K & 3) || N1 != 128 || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    const int64_t rows64 = (int64_t)B * Hh * Ww;
    if (rows64 > 0x7fffffffLL / 2) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(w1prep)) return SPGT_ERR_ALIGN;
    TcDense ld;
    ld.x = x; ld.lda = K; ld.rows = (int)rows64; ld.K = K;
    TcHeadEpi ep{b1, w2, b2, scale, shift, scale_map, shift_map, dirichlet, Hh, Ww, act, out};
    const int kpad = ceil_div(K, TC_BK) * TC_BK;
    return tc_launch<128, TcDense, EPI_HEAD, TcHeadEpi>(ld, (const float*)w1prep, kpad, (int)rows64, 1, ep, (cudaStream_t)stream);
}
