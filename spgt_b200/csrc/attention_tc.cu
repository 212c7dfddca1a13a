// Galerkin linear attention on the 5th-generation tensor cores (tcgen05, operands and accumulators in TMEM).
//
//   T[i][j]   = (1/S) * sum_s K[i][s] * V[j][s]        phase A: M = i, N = j, reduction over the grid nodes s
//   out[s][j] = sum_i Q[i][s] * T[i][j]                 phase B: M = s, N = j, reduction over i (dpk, zero padded to 40)
//
// Both contractions are 3xTF32 (x = hi + lo, three MMAs) so the result keeps fp32-level accuracy.  One cluster of
// 1-8 CTAs works on a (batch, head); each CTA streams its share of the S columns exactly once.
//
// Loads.  Rows of Q, K and V are only 4-byte aligned (S is arbitrary), and the number of bytes a CTA can keep in
// flight, not the instruction rate, limits the stream.  Every row piece is therefore fetched as 16-byte cp.async
// chunks that start at the aligned element at or below the first wanted column; the wanted columns then sit
// shift(row) = (element index of the row start) mod 4 floats into the shared-memory row, and the readers add that
// shift.  Piece starts are multiples of 32 columns, so the shift depends on the row only.
//
//   phase A  loader warps fill a deep ring of raw K / V sub-tiles (32 columns, 7 stages ~ 70 KB in flight);
//            converter warps split V into the hi / lo B operands (128B-swizzled K-major tiles, 2 stages) and move
//            the K rows - one row per thread - into TENSOR MEMORY as the hi / lo A operands; two issuing warps
//            multiply (128 x 48 x 8, A from TMEM, B from smem), each into its own accumulator.
//   reduce   the dpk x dpk partial sums of the cluster's CTAs are added in rank order through distributed shared
//            memory (deterministic, no global scratch), scaled by 1/S and written as the B operand of phase B.
//   phase B  Q tiles (128 grid nodes) are prefetched two tiles ahead into shared memory; 128 threads own one grid
//            node each: read its column, split, tcgen05.st into TMEM (A operand); the accumulator rows go back
//            through shared memory and leave as coalesced stores.
// warps 0-3 loaders / Q producers, 4-7 converters / epilogue, 8-9 MMA issuers.  Two CTAs fit per SM (256 TMEM columns,
// ~104 KB shared memory each).  Every wait is a bounded mbarrier poll that records an error code on expiry.
#include "tc_common.cuh"

namespace spgt {

__device__ int g_attn_status = 0;


constexpr int AT_THREADS = 320;                 // warps 0-3 loaders, 4-7 converters, 8-9 MMA issuers
constexpr int AT_NP = 48;                       // N (and B-tile rows) padded to a multiple of 16
constexpr int AT_SUB = 32;                      // columns per phase-A stage
constexpr int AT_FLUSH = 16;                    // sub-tiles whose products one tensor-memory accumulator sums before it is flushed
constexpr int AT_NR = 7;                        // raw K / V stages
constexpr int AT_RROWS = 36;                    // rows allocated per raw matrix (dpk <= 35)
constexpr int AT_RP = 36;                       // floats per raw row: 32 wanted + up to 3 of shift, in 16-byte chunks
constexpr int AT_RAW_MAT = AT_RROWS * AT_RP * 4;
constexpr int AT_RAW_STAGE = 2 * AT_RAW_MAT;    // K raw | V raw
constexpr int AT_TILE = AT_NP * 128;            // one K-major operand image: 48 rows x 128 bytes
constexpr int AT_QP = 132;                      // floats per Q row of a phase-B tile: 128 wanted + shift, 33 chunks
constexpr int AT_QSTAGE = AT_RROWS * AT_QP * 4;
constexpr int AT_NQ = 3;                        // Q stages (prefetch distance 2)
constexpr int AT_OUT_BYTES = 4 * 32 * 36 * 4;   // output staging of the four epilogue warps
constexpr int AT_RING_A = AT_NR * AT_RAW_STAGE;
constexpr int AT_RING_B = AT_NQ * AT_QSTAGE + AT_OUT_BYTES;
constexpr int AT_RING = ((AT_RING_A > AT_RING_B ? AT_RING_A : AT_RING_B) + 1023) / 1024 * 1024;
constexpr int AT_OP_OFF = AT_RING;              // phase A: 2 x (V hi | V lo); phase B: T images [k-block 0 hi | lo | k-block 1 hi | lo]
constexpr int AT_TC_OFF = AT_OP_OFF + 4 * AT_TILE;
constexpr int AT_TP = 36;                       // pitch of the dpk x dpk partial sums
constexpr int AT_SH_OFF = AT_TC_OFF + AT_TP * AT_TP * 4;   // shift table, 36 ints
constexpr int AT_BAR_OFF = AT_SH_OFF + 160;
constexpr int AT_SMEM_BYTES = 1024 + AT_BAR_OFF + 320;
constexpr int AT_TMEM_COLS = 256;
constexpr int AT_A1_COL = 96;                   // phase A: two accumulators at [0,48) and [48,96), two A stages (64 cols each) from here
constexpr int AT_A2_COL = 96;                   // phase B: accumulators at [0,48) and [48,96), A stages (80 cols) from here
static_assert(2 * (AT_SMEM_BYTES + 1024) <= 227 * 1024, "two CTAs per SM");

// 16-byte cp.async that reads `bytes` (0, 4, 8, 12 or 16) from the aligned source and zero-fills the rest
__device__ __forceinline__ void at_cp16(uint32_t dst, const float* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 2)
galerkin_attn_tc_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                        float* __restrict__ out, float* __restrict__ t_out, int S, int H, int merged) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* opr = smem + AT_OP_OFF;
    float* Tc = reinterpret_cast<float*>(smem + AT_TC_OFF);
    int* sh_tab = reinterpret_cast<int*>(smem + AT_SH_OFF);
    uint8_t* bar_mem = smem + AT_BAR_OFF;
    const uint32_t bars = smem_u32(bar_mem);
    auto raw_full = [&](int s) { return bars + 8u * s; };            // [7] loaders -> converters
    auto raw_empty = [&](int s) { return bars + 8u * (7 + s); };     // [7] converters -> loaders
    auto op_full = [&](int s) { return bars + 8u * (14 + s); };      // [2] converters -> MMA issuers
    auto op_empty = [&](int s) { return bars + 8u * (16 + s); };     // [2] MMA commits -> converters
    const uint32_t t_done = bars + 8u * 18;                          //     MMA commits -> T readout
    auto a2_full = [&](int s) { return bars + 8u * (19 + s); };      // [2] Q producers -> MMA
    auto a2_empty = [&](int s) { return bars + 8u * (21 + s); };     // [2] MMA commit -> Q producers
    auto d_full = [&](int b) { return bars + 8u * (23 + b); };       // [2] MMA commit -> epilogue
    auto d_empty = [&](int b) { return bars + 8u * (25 + b); };      // [2] epilogue -> MMA
    const uint32_t acc_free = bars + 8u * 27;                        //     T flush done -> MMA issuers
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mem + 256);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 264);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t C = cluster_nctarank();
    const uint32_t rank = cluster_ctarank();
    const int64_t bh = blockIdx.x / C;
    const int64_t e_bh = bh * (int64_t)D * S;                        // element index of this (batch, head) in Q / K / V
    const int sh_bh = (int)(e_bh & 3);                               // its offset from the 16-byte aligned element below it
    const float* Kb = K + (e_bh - sh_bh);
    const float* Vb = V + (e_bh - sh_bh);
    const float* Qb = Q + (e_bh - sh_bh);

    const int nsub = (S + AT_SUB - 1) / AT_SUB;
    const int sub_begin = (int)(((int64_t)rank * nsub) / C);
    const int sub_end = (int)(((int64_t)(rank + 1) * nsub) / C);
    const int nmine = sub_end - sub_begin;

    if (tid == 0) {
        for (int s = 0; s < AT_NR; ++s) { mbar_init(raw_full(s), 128); mbar_init(raw_empty(s), 128); }
        for (int s = 0; s < 2; ++s) { mbar_init(op_full(s), 128); mbar_init(op_empty(s), 2); }
        mbar_init(t_done, 2);
        mbar_init(acc_free, D > 32 ? 64 : 32);
        for (int s = 0; s < 2; ++s) { mbar_init(a2_full(s), 128); mbar_init(a2_empty(s), 1); mbar_init(d_full(s), 1); mbar_init(d_empty(s), 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(AT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid < AT_RROWS) sh_tab[tid] = tid < D ? ((sh_bh + tid * S) & 3) : 0;
    for (int i = tid; i < AT_TP * AT_TP; i += AT_THREADS) Tc[i] = 0.0f;
    for (int i = tid; i < 4 * AT_TILE / 16; i += AT_THREADS)            // rows of the V tiles beyond dpk are never written: keep them finite
        reinterpret_cast<uint4*>(opr)[i] = make_uint4(0u, 0u, 0u, 0u);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    constexpr uint32_t idesc = tc_idesc(AT_NP);

    // ============================== phase A: partial T over my columns ==============================
    if (warp < 4) {
        // The chunks a thread copies are the same for every sub-tile: (matrix, row, chunk) of index tid + 128 n.
        constexpr int NCH = 2 * D * 9;                                   // 16-byte chunks of one stage: K rows then V rows
        constexpr int NPT = (NCH + 127) / 128;
        const float* cbase[NPT];                                         // aligned source of the chunk for sub-tile column 0
        int crem[NPT];                                                   // elements from there to the end of the row
        uint32_t cdst[NPT];                                              // destination offset inside a raw stage
#pragma unroll
        for (int n = 0; n < NPT; ++n) {
            const int idx = tid + 128 * n;
            const bool in = idx < NCH;
            const int mat = idx >= D * 9 ? 1 : 0;
            const int j = in ? idx - mat * D * 9 : 0;
            const int row = j / 9, ch = j - 9 * row;
            const int e_row = sh_bh + row * S;
            const int start = (e_row & ~3) + 4 * ch;
            cbase[n] = (mat ? Vb : Kb) + start;
            crem[n] = in ? e_row + S - start : 0;
            cdst[n] = (uint32_t)(mat * AT_RAW_MAT + row * (AT_RP * 4) + ch * 16);
        }
        for (int it = 0; it < nmine; ++it) {
            const uint32_t st = (uint32_t)(it % AT_NR), ph = (uint32_t)((it / AT_NR) & 1);
            if (!mbar_wait(raw_empty(st), ph ^ 1, abort_flag, 1, &g_attn_status)) break;
            const int s0 = (sub_begin + it) * AT_SUB;
            const uint32_t dst0 = smem_base + st * AT_RAW_STAGE;
#pragma unroll
            for (int n = 0; n < NPT; ++n) {
                if (tid + 128 * n < NCH) {
                    int valid = crem[n] - s0;
                    valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
                    at_cp16(dst0 + cdst[n], valid > 0 ? cbase[n] + s0 : Kb, valid * 4);
                }
            }
            asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(raw_full(st)) : "memory");
        }
        cp_async_wait_all();
    } else if (warp < 8) {
        const int t = tid - 128, q = warp & 3;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const int krow = q * 32 + lane;                                 // K row moved to TMEM by this thread (q < 2)
        const bool k_warp = q * 32 < D;                                 // this warp owns at least one valid K row
        const int krow_rd = krow < AT_RROWS ? krow : AT_RROWS - 1;      // lanes beyond dpk read an allocated row; their TMEM lanes are never used
        const int ksh = sh_tab[krow_rd];
        // The V operand is converted by the warps that own no K row (the K warps' conversion of one row per thread is the
        // longest chain of a sub-tile): NV threads, eight per row, VN rows each.
        constexpr int NKQ = (D + 31) / 32, NV = (4 - NKQ) * 32, VR = NV / 8, VN = (D + VR - 1) / VR;
        const int tv = t - NKQ * 32;                                    // index among the V threads (negative: a K warp)
        int vrow[VN], vsh[VN];
#pragma unroll
        for (int n = 0; n < VN; ++n) { vrow[n] = (tv >> 3) + VR * n; vsh[n] = (tv >= 0 && vrow[n] < D) ? sh_tab[vrow[n]] : 0; }
        uint32_t st = 0, ph = 0;                                      // raw ring position, advanced without division
        for (int it = 0; it < nmine; ++it, st = (st + 1 == AT_NR ? 0u : st + 1), ph ^= (st == 0 ? 1u : 0u)) {
            const uint32_t so = (uint32_t)(it & 1), po = (uint32_t)((it >> 1) & 1);
            if (k_warp && it > 0 && it % AT_FLUSH == 0) {
                // The accumulate step of an MMA truncates, so the error of one long chain grows with its length (worst for
                // the all-positive position rows).  Every AT_FLUSH sub-tiles the two accumulators are added to the fp32
                // partial sum in shared memory with ordinary additions and the issuers start a new chain.
                if (!mbar_wait(t_done, (uint32_t)((it / AT_FLUSH - 1) & 1), abort_flag, 4, &g_attn_status)) break;
                tc_fence_after();
#pragma unroll 1
                for (int a = 0; a < 2; ++a) {                        // the two issuers' accumulators, one after the other
                    float v[32], w[16];
                    tc_ld32(tmem_base + lane_addr + a * AT_NP, v);
                    tc_ld16(tmem_base + lane_addr + a * AT_NP + 32, w);
                    if (a == 1) { tc_fence_before(); mbar_arrive(acc_free); }
                    if (krow < D) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (j < D) Tc[krow * AT_TP + j] += v[j];
#pragma unroll
                        for (int j = 0; j < 16; ++j) if (32 + j < D) Tc[krow * AT_TP + 32 + j] += w[j];
                    }
                }
            }
            if (!mbar_wait(raw_full(st), ph, abort_flag, 2, &g_attn_status)) break;
            // The operand stage is free once the MMAs two sub-tiles back are done.  The question is asked here, the answer is needed
            // only before the first store: the splits below run while it is on its way.
            const uint32_t op_ok = mbar_test_wait(op_empty(so), po ^ 1);
            const float* kraw = reinterpret_cast<const float*>(smem + st * AT_RAW_STAGE);
            const float* vraw = kraw + AT_RROWS * AT_RP;
            uint8_t* vhi = opr + so * (2 * AT_TILE);
            uint8_t* vlo = vhi + AT_TILE;
            if (!k_warp) {
                // V: raw rows -> hi / lo B operands (row = j, 32 k-values = grid nodes, 128B swizzle)
                uint32_t h[VN][4], l[VN][4];
#pragma unroll
                for (int n = 0; n < VN; ++n) {
                    if (vrow[n] < D) {
                        const float* p = vraw + vrow[n] * AT_RP + vsh[n] + 4 * (tv & 7);
#pragma unroll
                        for (int e = 0; e < 4; ++e) split_tf32_rn(p[e], h[n][e], l[n][e]);
                    }
                }
                if (!op_ok && !mbar_wait(op_empty(so), po ^ 1, abort_flag, 9, &g_attn_status)) break;
#pragma unroll
                for (int n = 0; n < VN; ++n) {
                    if (vrow[n] < D) {
                        const uint32_t off = tc_swz(vrow[n], tv & 7);
                        *reinterpret_cast<uint4*>(vhi + off) = make_uint4(h[n][0], h[n][1], h[n][2], h[n][3]);
                        *reinterpret_cast<uint4*>(vlo + off) = make_uint4(l[n][0], l[n][1], l[n][2], l[n][3]);
                    }
                }
            } else {
                // K: one row per thread into tensor memory (stage `so`, freed together with the V operands)
                const uint32_t a_hi = tmem_base + lane_addr + AT_A1_COL + so * 64;
                const float* p = kraw + krow_rd * AT_RP + ksh;
                bool ok = true;
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) split_tf32(p[16 * h2 + j], hi[j], lo[j]);
                    if (h2 == 0) {
                        if (!op_ok && !mbar_wait(op_empty(so), po ^ 1, abort_flag, 9, &g_attn_status)) { ok = false; break; }
                        tc_fence_after();
                    }
                    tc_st16(a_hi + 16 * h2, hi);
                    tc_st16(a_hi + 32 + 16 * h2, lo);
                }
                if (!ok) break;
            }
            mbar_arrive(raw_empty(st));                                 // this thread has read the raw stage
            if (k_warp) { tc_wait_st(); tc_fence_before(); }
            else fence_proxy_async();                                   // the V tiles were written with ordinary stores
            mbar_arrive(op_full(so));
        }
    } else {
        // Two issuing warps (one thread issues an MMA only about every 54 cycles; a 128 x 48 x 8 MMA takes 24): warp 8
        // multiplies k-steps 0-1 of every sub-tile into the accumulator at column 0, warp 9 k-steps 2-3 into the one at
        // column 48; the two partial sums are added when T is read out.
        const int iw = warp - 8;
        const uint32_t d = tmem_base + (uint32_t)(iw * AT_NP);
        for (int it = 0; it < nmine; ++it) {
            const uint32_t so = (uint32_t)(it & 1), po = (uint32_t)((it >> 1) & 1);
            if (it > 0 && it % AT_FLUSH == 0 &&
                !mbar_wait(acc_free, (uint32_t)((it / AT_FLUSH - 1) & 1), abort_flag, 10, &g_attn_status)) break;   // the flushed accumulator has been read
            if (!mbar_wait(op_full(so), po, abort_flag, 3, &g_attn_status)) break;
            tc_fence_after();
            if (lane == 0) {
                const uint32_t vhi = smem_base + AT_OP_OFF + so * (2 * AT_TILE);
                const uint64_t dbh = tc_smem_desc(vhi), dbl = tc_smem_desc(vhi + AT_TILE);
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    const int k8 = 2 * iw + kk;
                    const uint32_t ah = tmem_base + AT_A1_COL + so * 64 + k8 * 8, al = ah + 32;
                    const uint64_t adv = (uint64_t)(k8 * 2);
                    tc_mma_tf32_ts(d, al, dbh + adv, idesc, (it % AT_FLUSH != 0 || kk > 0) ? 1u : 0u);
                    tc_mma_tf32_ts(d, ah, dbl + adv, idesc, 1u);
                    tc_mma_tf32_ts(d, ah, dbh + adv, idesc, 1u);
                }
                tc_commit(op_empty(so));
                if (it == nmine - 1 || (it + 1) % AT_FLUSH == 0) tc_commit(t_done);
            }
            __syncwarp();
        }
    }

    // ============================== reduce T over the cluster ==============================
    if (warp >= 4 && warp < 8) {
        const int q = warp & 3;
        if (q * 32 < D) {                                               // warps that hold valid rows of T
            float v[32], w[16];
            bool have = false;
            if (nmine > 0) have = mbar_wait(t_done, (uint32_t)(((nmine - 1) / AT_FLUSH) & 1), abort_flag, 4, &g_attn_status);
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
                for (int j = 0; j < 32; ++j) if (j < D && have) Tc[row * AT_TP + j] += v[j];
#pragma unroll
                for (int j = 0; j < 16; ++j) if (32 + j < D && have) Tc[row * AT_TP + 32 + j] += w[j];
            }
        }
    }
    tc_fence_before();
    cluster_sync_all();        // every CTA's Tc is complete and all MMAs of phase A are done; also a CTA-wide barrier
    tc_fence_after();
    for (int i = tid; i < 4 * AT_TILE / 16; i += AT_THREADS)            // the T images reuse the V operand ring; their k padding must be zero
        reinterpret_cast<uint4*>(opr)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    {
        const float inv_s = 1.0f / (float)S;
        for (int e = tid; e < D * D; e += AT_THREADS) {
            const int i = e / D, j = e % D;
            float s = 0.0f;
            for (uint32_t r = 0; r < C; ++r) s += ld_dsmem_f32(Tc + i * AT_TP + j, r);
            s *= inv_s;
            if (t_out != nullptr && rank == 0) t_out[bh * D * D + e] = s;
            uint32_t hi, lo;
            split_tf32_rn(s, hi, lo);
            // B operand of phase B: row j (N), k = i; k-block i / 32
            uint8_t* img = opr + (i >> 5) * (2 * AT_TILE);
            const uint32_t off = tc_swz(j, (i & 31) >> 2) + (uint32_t)(i & 3) * 4u;
            *reinterpret_cast<uint32_t*>(img + off) = hi;
            *reinterpret_cast<uint32_t*>(img + AT_TILE + off) = lo;
        }
    }
    fence_proxy_async();
    __syncthreads();

    // ============================== phase B: out = Q^T T over my columns ==============================
    const int col_begin = sub_begin * AT_SUB;
    const int col_end = min(sub_end * AT_SUB, S);
    const int ntile = (col_end - col_begin + 127) / 128;
    const int64_t b_idx = bh / H, h_idx = bh % H;
    float* out_stage = reinterpret_cast<float*>(smem + AT_NQ * AT_QSTAGE);
    if (warp < 4) {
        const int q = warp & 3;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        // Q tile loader.  Thread (w = warp, ch = lane) copies chunk ch of rows w, w + 4, w + 8, ...: rows four apart
        // have the same shift, so their aligned sources are exactly 4 S floats apart and share the valid-byte count.
        // The 33rd chunk of every row (needed when the shift is not zero) is copied by threads 0 .. dpk-1.
        const int e_w = sh_bh + warp * S;
        const float* qsrc0 = Qb + (e_w & ~3) + 4 * lane;
        const int qrem0 = S + (e_w & 3) - 4 * lane;                      // elements from chunk `lane` of column 0 to the row end
        const int e_x = sh_bh + (tid < D ? tid : 0) * S;
        const float* xsrc0 = Qb + (e_x & ~3) + 128;
        const int xrem0 = S + (e_x & 3) - 128;
        auto load_q = [&](int tile) {
            if (tile < ntile) {
                const int c0 = col_begin + tile * 128;
                const uint32_t dst0 = smem_base + (uint32_t)(tile % AT_NQ) * AT_QSTAGE;
                int valid = qrem0 - c0;
                valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
                const float* src = valid > 0 ? qsrc0 + c0 : Qb;
                const size_t step = valid > 0 ? (size_t)4 * S : 0;
                uint32_t dst = dst0 + warp * (AT_QP * 4) + lane * 16;
#pragma unroll
                for (int k = 0; k < (D + 3) / 4; ++k) {
                    if (warp + 4 * k < D) at_cp16(dst, src, valid * 4);
                    src += step;
                    dst += 4 * AT_QP * 4;
                }
                if (tid < D) {
                    int vx = xrem0 - c0;
                    vx = vx < 0 ? 0 : (vx > 4 ? 4 : vx);
                    at_cp16(dst0 + tid * (AT_QP * 4) + 32 * 16, vx > 0 ? xsrc0 + c0 : Qb, vx * 4);
                }
            }
            cp_async_commit();                                           // one group per tile slot, empty past the end
        };
        const int s4 = S & 3;
        load_q(0);
        load_q(1);
        bool alive = true;                                               // after a failed wait keep meeting the others at the barrier
        for (int it = 0; it < ntile; ++it) {
            const uint32_t sa = (uint32_t)(it & 1), ph = (uint32_t)((it >> 1) & 1);
            cp_async_wait<1>();                                          // my chunks of tile `it` have landed
            asm volatile("bar.sync 1, 128;" ::: "memory");              // ... and everyone else's; tile it-1 has been read by all
            load_q(it + 2);                                              // into the stage tile it-1 used
            if (!alive) continue;
            const int s = col_begin + it * 128 + tid;
            const bool ok = s < col_end;
            const float* qs = reinterpret_cast<const float*>(smem + (it % AT_NQ) * AT_QSTAGE) + tid;
            float qv[40];
#pragma unroll
            for (int i = 0; i < 40; ++i) qv[i] = (i < D && ok) ? qs[i * AT_QP + ((sh_bh + i * s4) & 3)] : 0.0f;
            if (!mbar_wait(a2_empty(sa), ph ^ 1, abort_flag, 5, &g_attn_status)) { alive = false; continue; }
            tc_fence_after();
            const uint32_t a_hi = tmem_base + lane_addr + AT_A2_COL + sa * 80, a_lo = a_hi + 40;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) split_tf32(qv[16 * c + j], hi[j], lo[j]);
                tc_st16(a_hi + 16 * c, hi);
                tc_st16(a_lo + 16 * c, lo);
            }
            {
                uint32_t hi[8], lo[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) split_tf32(qv[32 + j], hi[j], lo[j]);
                tc_st8(a_hi + 32, hi);
                tc_st8(a_lo + 32, lo);
            }
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(a2_full(sa));
        }
        cp_async_wait_all();
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
                    const uint32_t img = smem_base + AT_OP_OFF + (k8 >> 2) * (2 * AT_TILE);
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
    static SmemOptIn configured;
    auto kern = galerkin_attn_tc_kernel<D>;
    if (int e = smem_opt_in(kern, AT_SMEM_BYTES, configured)) return e;
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


int attn_tc_status_reset() {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int)) == cudaSuccess ? SPGT_OK : SPGT_ERR_LAUNCH;
}

int attn_tc_status() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)) != cudaSuccess) return SPGT_ERR_LAUNCH;
    return v;
}

}  // namespace spgt
