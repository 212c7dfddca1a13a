// Dense contractions on the 5th-generation tensor cores (tcgen05) with 3xTF32:
//   C[rows, N] = A[rows, K] * W[K, N],   A*W ~= A_lo*W_hi + A_hi*W_lo + A_hi*W_hi   (fp32-level accuracy).
//
// Persistent, warp-specialised kernel, one CTA (576 or 608 threads) per SM.  A 128 x 128 x 8 tf32 MMA with both operands
// in shared memory already consumes the whole shared-memory bandwidth of an SM, and 3xTF32 reads every operand
// twice, so the operands are kept off that path:
//   * A (activations) is an MMA operand in TENSOR MEMORY: loader warps cp.async the raw fp32 tile (dense rows, or
//     the implicit-GEMM gather of a 3x3 convolution) with fully coalesced 16-byte copies into a 128B-swizzled
//     staging ring; splitter threads own one row each, read it back conflict-free, split it into tf32 hi / lo and
//     write both into TMEM with tcgen05.st.  (Loading one row per thread straight from global memory was tried:
//     its 32 lines per load instruction saturate the L1 miss path and slow every other memory access of the SM.)
//   * W is prepared once (split, transposed to K-major, 128B-swizzled tile images) and arrives by one
//     cp.async.bulk per k-block; when a whole column tile of W fits the ring it stays resident for the kernel.
//   * Accumulators live in TMEM.  MT = 1: one 128-row tile with double-buffered accumulators (the epilogue of a
//     tile overlaps the MMAs of the next).  MT = 2: two 128-row tiles share every W stage (halves the L2 traffic of
//     W for long-K problems such as the 3x3 convolutions).
//   * Row-major epilogues stage each thread's row in padded shared memory and leave as warp-cooperative coalesced
//     float4 stores (full 128-byte lines, residual added on the way); the projection epilogue does the per-head
//     LayerNorm thread-locally and stores head-major through the same staging; the decoder head keeps its
//     constants in shared memory and reduces its row dot product across the two column halves.  Whatever an
//     epilogue reads from global memory (residual, position values, de-normalisation maps) is fetched one phase
//     ahead, while the accumulator is still being computed.
//   * Column tiles of up to 64 use two MMAs per k-step instead of three: A_hi * [W_hi | W_lo] as one instruction of
//     twice the width into two partial accumulators, A_lo * W_hi into the first.
//   warps 0-3 A loaders, 4-7 A splitters, 8 W loader, 9 (MT = 2: 9-10) MMA issuers (lane 0 runs the whole issue loop),
//   then 8 epilogue warps.
// All waits are bounded mbarrier polls: on expiry the kernel records an error code, stops waiting and returns.
#include "tc_common.cuh"

namespace spgt {

constexpr int TC_BLOAD_WARP = 8, TC_MMA_WARP = 9, TC_EPI_WARPS = 8;
// MMA-issuing warps: two with two row tiles per unit (one tile each), one otherwise; the epilogue warps follow them
__host__ __device__ constexpr int tc_mma_warps(int mt) { return mt == 2 ? 2 : 1; }
__host__ __device__ constexpr int tc_epi_warp0(int mt) { return TC_MMA_WARP + tc_mma_warps(mt); }
__host__ __device__ constexpr int tc_threads(int mt, int epi_groups = 1) { return 32 * (tc_epi_warp0(mt) + epi_groups * TC_EPI_WARPS); }

__device__ int g_tc_status = 0;          // 0 = ok; otherwise the code of the first wait that gave up


__host__ __device__ constexpr int tc_cols_per_thread(int bn, int mt, bool colsplit = false) { return (mt == 1 ? bn / 2 : bn) / (colsplit ? 2 : 1); }

// Position in a ring of N stages: stage index and the parity of the pass, advanced without division.
struct TcRing {
    uint32_t s = 0, ph = 0;
    template <int N> __device__ __forceinline__ void next() { if (++s == (uint32_t)N) { s = 0; ph ^= 1u; } }
    __device__ __forceinline__ void next_of(uint32_t n) { if (++s == n) { s = 0; ph ^= 1u; } }
};

// ---- A-operand loaders.  A loader thread copies 16-byte chunk (t & 7) of rows (t >> 3) + 16 i of every tile:
// per-row state is computed once per work unit, per-k-block state once per k-block.
// Every loader also says where a work unit's W stages come from (w_src; W_PER_UNIT = true: another image per unit, W is
// then streamed and never resident), which output row a GEMM row is stored to (out_row; -1 = padding row, not stored), and
// whether the splitter threads read a row of the raw tile each (the tile rows are the GEMM rows) or a column each
// (COLUMN_SPLIT: the tile holds A transposed, 32 k-values as its rows).
// Ring depths, 0 = the default of the tile shape: RAW_STAGES raw A stages and W_STAGES W stages in shared memory, A_STAGES A
// stages in tensor memory.  STAGING = false: the epilogue needs no shared-memory staging rows.  CONST_A: the A operand of
// the LAST k-block is the same for every work unit and stays in tensor memory (the loader's const_row() gives its rows);
// REVERSE_UNITS: work units are taken from the last to the first.
// W_CONVERT: the W stage of the last k-block is not copied from a prepared image but split and laid out by the W-loader
// warp from a plain [w_plain_rows()][32] fp32 block per unit (w_plain(unit)), so the producer of that block can store it
// coalesced and it takes no more memory than its values.  ACC_BUFS: accumulator buffers (0 = default of the tile shape).
struct TcLoaderDefaults {
    static constexpr bool W_PER_UNIT = false, COLUMN_SPLIT = false, STAGING = true, CONST_A = false, REVERSE_UNITS = false, W_CONVERT = false;
    static constexpr int RAW_STAGES = 0, W_STAGES = 0, A_STAGES = 0, ACC_BUFS = 0;
    // Groups of eight epilogue warps.  With two, group g finishes the units whose accumulator buffer is g (every second
    // unit), so one unit's activation and stores overlap the next unit's: for short k, where the epilogue is the longest stage.
    static constexpr int EPI_GROUPS = 1;
    // Two groups working on the same unit instead (two row tiles of 128 columns only): a thread finishes half of its row's
    // columns, so the accumulator is held for a shorter time; for long k with one accumulator buffer, where the MMAs wait for
    // the epilogue.  (With 64-wide tiles the extra warps slowed the producers down more than the epilogue gained.)
    static constexpr bool EPI_COLSPLIT = false;
    static constexpr bool RESIDUAL = true;        // false: the LINEAR epilogue's residual path is compiled out
    // With W_CONVERT and two k-blocks: the prepared image of the first k-block is the same for every unit and stays in the
    // last W stage (loaded once), the ring of the other stages carries the converted blocks only.
    static constexpr bool W_TAIL_RESIDENT = false;
    __device__ __forceinline__ const float* const_row(int) const { return nullptr; }
    __device__ __forceinline__ const float* w_plain(int) const { return nullptr; }
    __device__ __forceinline__ int w_plain_rows() const { return 0; }
    __device__ __forceinline__ int const_ksteps() const { return TC_BK / 8; }     // k-steps of 8 the constant A block really has
};
struct TcDense : TcLoaderDefaults {
    const float* x; int lda; int rows; int K;
    __device__ __forceinline__ const float* w_src(const float* wtile, int, int kb, int stage_floats) const { return wtile + (int64_t)kb * stage_floats; }
    __device__ __forceinline__ int64_t out_row(int row) const { return row < rows ? row : -1; }
    __device__ __forceinline__ int out_valid(int row0) const { return rows - row0; }
    struct Row { const float* p; bool ok; };
    struct Kst { int kc; bool ok; };
    __device__ __forceinline__ Row row_state(int row) const {
        Row r; r.ok = row < rows; r.p = x + (int64_t)(r.ok ? row : 0) * lda; return r;
    }
    __device__ __forceinline__ Kst k_state(int kb, int chunk) const {
        Kst k; k.kc = kb * TC_BK + chunk * 4; k.ok = k.kc < K; if (!k.ok) k.kc = 0; return k;
    }
    __device__ __forceinline__ const float* ptr(const Row& r, const Kst& k, bool& ok) const { ok = r.ok && k.ok; return r.p + k.kc; }
};
struct TcConv : TcLoaderDefaults {          // 3x3, padding 1, NHWC; k = tap * Cin + c with Cin % 4 == 0
    static constexpr bool EPI_COLSPLIT = true;
    const float* x; int cin_pitch, cin_off, Cin, Hh, Ww; int rows; int K;
    __device__ __forceinline__ const float* w_src(const float* wtile, int, int kb, int stage_floats) const { return wtile + (int64_t)kb * stage_floats; }
    __device__ __forceinline__ int64_t out_row(int row) const { return row < rows ? row : -1; }
    __device__ __forceinline__ int out_valid(int row0) const { return rows - row0; }
    struct Row { const float* p; uint32_t mask; };     // bit tap of mask: the tap's source pixel lies inside the image
    struct Kst { int off; int tap; };
    __device__ __forceinline__ Row row_state(int row) const {
        Row r; r.mask = 0; r.p = x;
        if (row < rows) {
            const int b = row / (Hh * Ww);
            const int rem = row - b * Hh * Ww;
            const int py = rem / Ww, px = rem - py * Ww;
            r.p = x + (int64_t)row * cin_pitch + cin_off;
#pragma unroll
            for (int tap = 0; tap < 9; ++tap) {
                const int yy = py + tap / 3 - 1, xx = px + tap % 3 - 1;
                if (yy >= 0 && yy < Hh && xx >= 0 && xx < Ww) r.mask |= 1u << tap;
            }
        }
        return r;
    }
    __device__ __forceinline__ Kst k_state(int kb, int chunk) const {
        Kst k;
        const int kk = kb * TC_BK + chunk * 4;
        k.tap = kk / Cin;                               // >= 9 in the zero padding of K: no mask bit is set there
        const int c = kk - k.tap * Cin;
        const int dy = k.tap / 3 - 1, dx = k.tap - (k.tap / 3) * 3 - 1;
        k.off = (dy * Ww + dx) * cin_pitch + c;
        return k;
    }
    __device__ __forceinline__ const float* ptr(const Row& r, const Kst& k, bool& ok) const {
        ok = (r.mask >> k.tap) & 1u;
        return ok ? r.p + k.off : x;
    }
};

// Spectral layer, inverse transform along y plus the residual linear layer, as one GEMM per image row (b, x):
//   out[y][o] = sum_i X[y][i] Wr[i][o] + sum_j F3[y][j] P[j][o]            K = 32 channels + 32 (the 2m <= 32 kept modes, zero padded)
// The GEMM rows of an image row are padded to `upr` units of 256 (two 128-row tiles): GEMM row R lies in unit u = R / 256,
// image row u / upr, y = (u % upr) * 256 + R % 256.  k-block 0 takes its A rows from X and its W stage from the prepared
// image of Wr; k-block 1 takes its A rows from the F3 table ([upr * 256][32], zero beyond r and beyond 2m) and its W
// stage from the image of the row's P block, which the x-transform kernel writes in the W stage layout.
struct TcSpecInv : TcLoaderDefaults {
    static constexpr bool W_PER_UNIT = true;
    const float* x; const float* f3; const float* wr_img; const float* p_img; int r, upr; int rows; int K;
    __device__ __forceinline__ const float* w_src(const float*, int unit, int kb, int stage_floats) const {
        return kb == 0 ? wr_img : p_img + (int64_t)(unit / upr) * stage_floats;
    }
    __device__ __forceinline__ int64_t out_row(int row) const {
        const int u = row >> 8, img = u / upr, y = (u - img * upr) * 256 + (row & 255);
        return (row < rows && y < r) ? (int64_t)img * r + y : -1;
    }
    __device__ __forceinline__ int out_valid(int row0) const {
        const int u = row0 >> 8, img = u / upr, y = (u - img * upr) * 256 + (row0 & 255);
        return row0 < rows ? r - y : 0;
    }
    struct Row { const float* px; const float* pf; bool ok; };
    struct Kst { int kb; int c4; };
    __device__ __forceinline__ Row row_state(int row) const {
        const int u = row >> 8, img = u / upr, y = (u - img * upr) * 256 + (row & 255);
        Row s; s.ok = row < rows && y < r;
        s.px = s.ok ? x + ((int64_t)img * r + y) * 32 : x;
        s.pf = f3 + (int64_t)y * 32;
        return s;
    }
    __device__ __forceinline__ Kst k_state(int kb, int chunk) const { Kst k; k.kb = kb; k.c4 = chunk * 4; return k; }
    __device__ __forceinline__ const float* ptr(const Row& s, const Kst& k, bool& ok) const {
        if (k.kb == 0) { ok = s.ok; return s.px + k.c4; }
        ok = true; return s.pf + k.c4;
    }
};
// The same for r <= 256 (one unit per image row): the F3 rows are the same for every image row, so they are split once
// and kept in tensor memory as the A operand of k-block 1; only X passes through the raw ring (four stages of 32 KB).
// The row's P block arrives as plain fp32 [J][32] and is laid out by the W-loader warp.  Tensor memory holds two
// accumulator buffers, one A stage and the constant block (measured: 222 us for 64 x 211 image rows against 281 us with one
// accumulator buffer and two A stages).  Image rows are taken from the last to the first: the ones the forward transform
// read last are the ones still in L2.
struct TcSpecInvC : TcLoaderDefaults {
    static constexpr bool W_PER_UNIT = true, CONST_A = true, REVERSE_UNITS = true, W_CONVERT = true;     // (W_CONVERT needs 32-wide column tiles: lane = image row)
    static constexpr int RAW_STAGES = 3, W_STAGES = 4, A_STAGES = 1, EPI_GROUPS = 2;
    static constexpr bool RESIDUAL = false, W_TAIL_RESIDENT = true;
    const float* x; const float* f3; const float* wr_img; const float* p; int J; int r; int rows; int K;
    __device__ __forceinline__ const float* w_src(const float*, int, int, int) const { return wr_img; }
    __device__ __forceinline__ const float* w_plain(int unit) const { return p + (int64_t)unit * J * 32; }
    __device__ __forceinline__ int w_plain_rows() const { return J; }
    __device__ __forceinline__ int const_ksteps() const { return (J + 7) / 8; }
    __device__ __forceinline__ int64_t out_row(int row) const {
        const int y = row & 255;
        return (row < rows && y < r) ? (int64_t)(row >> 8) * r + y : -1;
    }
    __device__ __forceinline__ int out_valid(int row0) const { return row0 < rows ? r - (row0 & 255) : 0; }
    __device__ __forceinline__ const float* const_row(int row_in_unit) const { return f3 + (int64_t)row_in_unit * 32; }
    struct Row { const float* px; bool ok; };
    struct Kst { int c4; };
    __device__ __forceinline__ Row row_state(int row) const {
        const int y = row & 255;
        Row s; s.ok = row < rows && y < r;
        s.px = s.ok ? x + ((int64_t)(row >> 8) * r + y) * 32 : x;
        return s;
    }
    __device__ __forceinline__ Kst k_state(int, int chunk) const { Kst k; k.c4 = chunk * 4; return k; }
    __device__ __forceinline__ const float* ptr(const Row& s, const Kst& k, bool& ok) const { ok = s.ok; return s.px + k.c4; }
};
// Spectral layer, forward transform along y: Y1[x][j][c] = sum_y F1[j][y] X[x][y][c] as the GEMM D[(x, c)][j] with
// A[(x, c)][k = y] = X[x][y][c].  A is stored transposed in memory (c contiguous), so a raw tile holds, for four image rows,
// 32 consecutive y as its rows (tile row = x_local * 32 + y_local, 32 channels each) and splitter thread (x_local, c)
// reads column c of the 32 tile rows of its image row.  W is the prepared image of F1^T ([y][j]).
struct TcSpecFwd : TcLoaderDefaults {
    // The kernel is bound by the bytes it keeps in flight: five raw stages of 32 KB; seven W stages keep the image of F1^T
    // resident up to r = 224; the epilogue stores straight from registers.
    static constexpr bool COLUMN_SPLIT = true, STAGING = false;
    static constexpr int RAW_STAGES = 5, W_STAGES = 7;
    const float* x; int r; int64_t nimg; int rows; int K;
    __device__ __forceinline__ const float* w_src(const float* wtile, int, int kb, int stage_floats) const { return wtile + (int64_t)kb * stage_floats; }
    __device__ __forceinline__ int64_t out_row(int row) const { return row < rows ? row : -1; }
    __device__ __forceinline__ int out_valid(int row0) const { return rows - row0; }
    struct Row { const float* p; int y; bool ok; };
    struct Kst { int kb; int c4; };
    __device__ __forceinline__ Row row_state(int row) const {
        const int64_t img = (int64_t)(row >> 7) * 4 + ((row & 127) >> 5);
        Row s; s.y = row & 31; s.ok = img < nimg;
        s.p = x + ((s.ok ? img : 0) * r + s.y) * 32;
        return s;
    }
    __device__ __forceinline__ Kst k_state(int kb, int chunk) const { Kst k; k.kb = kb; k.c4 = chunk * 4; return k; }
    __device__ __forceinline__ const float* ptr(const Row& s, const Kst& k, bool& ok) const {
        ok = s.ok && k.kb * TC_BK + s.y < r;
        return ok ? s.p + (int64_t)k.kb * (TC_BK * 32) + k.c4 : x;
    }
};

// ---- epilogue parameter blocks ------------------------------------------------------------------------------
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
struct TcSpecFwdEpi { float* y1; int J; int64_t nimg; };     // Y1 [image row][J][32 channels]
enum { EPI_LINEAR = 0, EPI_PROJ = 1, EPI_HEAD = 2, EPI_SPECF = 3 };

template <class Loader, int MT, int BN, int EPI = EPI_LINEAR> __host__ __device__ constexpr int tc_epi_groups() {
    if (EPI == EPI_HEAD) return MT == 1 ? 2 : 1;     // the decoder head: 128 activations per row and one k-block, the epilogue is the longest stage
    return Loader::EPI_COLSPLIT ? ((MT == 2 && BN == 128) ? 2 : 1) : Loader::EPI_GROUPS;
}

template <int BN, int MT, class Loader = TcDense, int EPI = EPI_LINEAR> struct TcCfg {
    // Column tiles of up to 64: W_hi and W_lo of a k-block lie one after the other in shared memory, so one MMA of
    // twice the width computes A_hi W_hi and A_hi W_lo side by side (two partial accumulators, summed by the epilogue)
    // and a k-step of 8 takes two MMA instructions instead of three; the issuing thread is what limits these tiles.
    static constexpr bool MERGE = BN <= 64;
    static constexpr int ACCW = MERGE ? 2 * BN : BN;                // accumulator columns of one row tile
    static constexpr int NBUF = Loader::ACC_BUFS ? Loader::ACC_BUFS : ((MT == 1 || ACCW <= 64) ? 2 : 1);    // accumulator buffers
    static constexpr int ACC_COLS = NBUF * MT * ACCW;
    static constexpr int SA = Loader::A_STAGES ? Loader::A_STAGES : ((MT == 1) ? 4 : 2);   // A stages in TMEM, 64 columns (hi|lo) per tile
    static constexpr int CONST_COLS = Loader::CONST_A ? MT * 64 : 0;                      // the constant A k-block (hi|lo per tile)
    static_assert(ACC_COLS + SA * MT * 64 + CONST_COLS <= 512, "tensor memory budget");
    static constexpr int B_BYTES = 2 * BN * TC_BK * 4;              // W_hi | W_lo image of one k-block
    static constexpr int SB = Loader::W_STAGES ? Loader::W_STAGES
                                               : ((BN == 128) ? (MT == 1 ? 4 : 3) : ((MT == 1 || BN == 32) ? 8 : 6));  // W stages in shared memory
    static constexpr int RAW_BYTES = MT * TC_BM * TC_BK * 4;        // raw fp32 A tile(s) of one k-block
    // Raw A stages in shared memory.  Epilogues without staging rows (PROJ, HEAD) spend that memory on two more stages: the
    // dense kernels are bound by the bytes they keep in flight.  At run time the stages of the W ring that a resident W does
    // not need are added to the raw ring as well (up to eight stages).
    static constexpr bool EPI_STAGING = Loader::STAGING && EPI == EPI_LINEAR;
    static constexpr int SR = Loader::RAW_STAGES ? Loader::RAW_STAGES : ((MT == 1) ? ((!EPI_STAGING && BN == 128) ? 5 : 3) : 2);
    static constexpr bool CS = Loader::EPI_COLSPLIT && MT == 2 && BN == 128;     // sixteen epilogue warps share every unit
    static constexpr int EG = tc_epi_groups<Loader, MT, BN, EPI>();
    static constexpr int CPT = tc_cols_per_thread(BN, MT, CS);      // columns an epilogue thread finishes
    static constexpr int PASS = CS ? 16 : (CPT > 32 ? (CPT % 32 == 0 ? 32 : 16) : CPT);    // columns per staging pass of the LINEAR epilogue
    static constexpr int SLOT_BYTES = PASS * 4 + 16;                // per-epilogue-thread staging row + 16 bytes (bank skew)
    static constexpr int STAGING_BYTES = EPI_STAGING ? 32 * EG * TC_EPI_WARPS * SLOT_BYTES : (EPI == EPI_HEAD ? 2048 : 0);   // (HEAD: [2 units][2 groups][128] partial row sums)
    static constexpr int CONST_BYTES = 2048;                        // per-CTA epilogue constants (bias, LayerNorm affine, head vectors)
    static constexpr int BAR_BYTES = 384;
    static constexpr int PLAIN_BYTES = Loader::W_CONVERT ? 4 * 32 * 32 * 4 : 0;       // ring of plain W blocks (after the barriers)
    static constexpr size_t BYTES = 1024 + (size_t)SB * B_BYTES + SR * RAW_BYTES + STAGING_BYTES + CONST_BYTES + BAR_BYTES + PLAIN_BYTES;
    static_assert(BYTES <= 227 * 1024, "shared memory budget");
};

template <int BN, int MT, class Loader, int EPI, class EpiParams>
__global__ void __launch_bounds__(tc_threads(MT, tc_epi_groups<Loader, MT, BN, EPI>()), 1)
tc_gemm_kernel(Loader ld, const float* __restrict__ wimg, int kpad, int rows, int n_tiles, int m_units, EpiParams ep) {
    using C = TcCfg<BN, MT, Loader, EPI>;
    constexpr int SA = C::SA, NBUF = C::NBUF, SR = C::SR;
    constexpr int SB = C::SB;
    constexpr uint32_t B_STAGE = C::B_BYTES;
    constexpr int NIWARPS = tc_mma_warps(MT);                       // MMA-issuing warps
    constexpr int EG = C::EG;
    constexpr bool CS = C::CS;
    constexpr int TC_THREADS = tc_threads(MT, EG), TC_EPI_WARP0 = tc_epi_warp0(MT);
    static_assert(EG == 1 || (EG == 2 && (CS || C::NBUF == 2) && (EPI == EPI_LINEAR || EPI == EPI_HEAD)), "two epilogue groups: one per accumulator buffer, or sharing every unit");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;          // 1024-aligned for the 128B swizzle
    uint8_t* smem = smem_raw + (smem_base - smem_u32(smem_raw));
    uint8_t* staging = smem + C::SB * C::B_BYTES + SR * C::RAW_BYTES;
    float* consts = reinterpret_cast<float*>(staging + C::STAGING_BYTES);
    uint8_t* bar_mem = staging + C::STAGING_BYTES + C::CONST_BYTES;
    const uint32_t bars = smem_u32(bar_mem);
    // barrier slots (8 bytes each)
    auto a_full = [&](int s) { return bars + 8u * s; };                 // [4]
    auto a_empty = [&](int s) { return bars + 8u * (4 + s); };          // [4]
    auto b_full = [&](int s) { return bars + 8u * (8 + s); };           // [8]
    auto b_empty = [&](int s) { return bars + 8u * (16 + s); };         // [8]
    auto acc_full = [&](int b) { return bars + 8u * (24 + b); };        // [2]
    auto acc_empty = [&](int b) { return bars + 8u * (26 + b); };       // [2]
    auto raw_full = [&](int s) { return bars + 8u * (28 + s); };        // [8]
    auto raw_empty = [&](int s) { return bars + 8u * (36 + s); };       // [8]
    static_assert(SA <= 4 && SB <= 8 && SR <= 8 && NBUF <= 2, "barrier slots");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_mem + 352);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bar_mem + 360);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int KB = kpad / TC_BK;
    const int KBA = Loader::CONST_A ? KB - 1 : KB;                   // k-blocks whose A operand passes through the rings
    const bool resident = !Loader::W_PER_UNIT && KB <= SB;          // the whole column tile of W stays in shared memory
    // Raw A ring (1024-aligned stages): it begins after the W stages in use, so a resident W of fewer than SB k-blocks
    // leaves its unused stages to the raw ring.
    const int sb_used = resident ? KB : SB;
    int sr_n = SR + ((SB - sb_used) * C::B_BYTES) / C::RAW_BYTES;
    if (sr_n > 8) sr_n = 8;
    const uint32_t SRn = (uint32_t)sr_n;
    uint8_t* raw = smem + sb_used * C::B_BYTES;

    if (tid == 0) {
        for (int s = 0; s < SA; ++s) { mbar_init(a_full(s), 128); mbar_init(a_empty(s), NIWARPS); }
        for (int s = 0; s < 8; ++s) { mbar_init(raw_full(s), 128); mbar_init(raw_empty(s), 128); }
        for (int s = 0; s < SB; ++s) { mbar_init(b_full(s), 1); mbar_init(b_empty(s), NIWARPS); }
        for (int b = 0; b < 2; ++b) { mbar_init(acc_full(b), NIWARPS); mbar_init(acc_empty(b), 32 * TC_EPI_WARPS * (CS ? 2 : 1)); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // Epilogue constants of this CTA's column tile go to shared memory once: a global load issued from the epilogue
    // queues behind the producers' traffic and costs microseconds of latency per use.
    if constexpr (EPI == EPI_SPECF) {
        // no epilogue constants
    } else if constexpr (EPI == EPI_HEAD) {
        for (int i = tid; i < 256; i += TC_THREADS) consts[i] = i < 128 ? __ldg(ep.b1 + i) : __ldg(ep.w2 + i - 128);
    } else if constexpr (EPI == EPI_LINEAR) {
        const int ntc = blockIdx.x % n_tiles;
        for (int i = tid; i < BN; i += TC_THREADS) {
            const int col = ntc * BN + i;
            consts[i] = (ep.bias != nullptr && col < ep.N) ? __ldg(ep.bias + col) : 0.0f;
        }
    } else {
        const int p = blockIdx.x % n_tiles;
        for (int i = tid; i < 128; i += TC_THREADS) {
            consts[i] = ep.bias[p] ? __ldg(ep.bias[p] + i) : 0.0f;
            consts[128 + i] = ep.lnw[p] ? __ldg(ep.lnw[p] + i) : 1.0f;
            consts[256 + i] = ep.lnb[p] ? __ldg(ep.lnb[p] + i) : 0.0f;
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_a = tmem_base + C::ACC_COLS;
    const uint32_t tmem_c = tmem_a + SA * MT * 64;                   // the constant A k-block, 64 columns (hi|lo) per tile
    if constexpr (Loader::CONST_A) {
        // the splitter warps write the constant A rows (one row of 32 floats per thread and tile) once
        if (warp >= 4 && warp < 8) {
            const int q = warp & 3;
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const float4* src = reinterpret_cast<const float4*>(ld.const_row(m * TC_BM + q * 32 + lane));
                const uint32_t dst = tmem_c + ((uint32_t)(q * 32) << 16) + m * 64;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 w = __ldg(src + 4 * h + j);
                        split_tf32(w.x, hi[4 * j], lo[4 * j]); split_tf32(w.y, hi[4 * j + 1], lo[4 * j + 1]);
                        split_tf32(w.z, hi[4 * j + 2], lo[4 * j + 2]); split_tf32(w.w, hi[4 * j + 3], lo[4 * j + 3]);
                    }
                    tc_st16(dst + 16 * h, hi);
                    tc_st16(dst + 32 + 16 * h, lo);
                }
            }
            tc_wait_st();
        }
        tc_fence_before();
        __syncthreads();
        tc_fence_after();
    }

    // Work distribution: this CTA keeps one column tile (so a resident W is loaded once) and strides over row units.
    const int sched_id = blockIdx.x, sched_n = gridDim.x;
    const int ctas_per_nt = sched_n / n_tiles;
    const int nt = sched_id % n_tiles;
    const int u0 = sched_id / n_tiles;
    const int n_my_units = (u0 < m_units) ? (m_units - u0 + ctas_per_nt - 1) / ctas_per_nt : 0;
    const float* wtile = wimg + (int64_t)nt * KB * (C::B_BYTES / 4);
    // index of this CTA's ui-th work unit, and its first row tile (MT tiles follow each other)
    auto unit_index = [&](int ui) { const int u = u0 + ui * ctas_per_nt; return Loader::REVERSE_UNITS ? m_units - 1 - u : u; };
    auto unit_tile0 = [&](int ui) { return unit_index(ui) * MT; };

    if (warp < 4) {
        // ------------------------------------------ A loaders ------------------------------------------
        const int t = tid;
        uint32_t aoff[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) aoff[i] = tc_swz((t >> 3) + 16 * i, t & 7);
        const uint32_t raw_s = smem_u32(raw);
        TcRing rr;
        bool alive = true;
        for (int ui = 0; ui < n_my_units && alive; ++ui) {
            const int row0 = unit_tile0(ui) * TC_BM + (t >> 3);
            typename Loader::Row rs[MT][8];
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int i = 0; i < 8; ++i) rs[m][i] = ld.row_state(row0 + m * TC_BM + 16 * i);
            for (int kb = 0; kb < KBA; ++kb, rr.next_of(SRn)) {
                const uint32_t sr = rr.s, ph = rr.ph;
                bool okw; okw = mbar_wait(raw_empty(sr), ph ^ 1, abort_flag, 1, &g_tc_status);
                if (!okw) { alive = false; break; }
                const typename Loader::Kst ks = ld.k_state(kb, t & 7);
                const uint32_t dst = raw_s + sr * C::RAW_BYTES;
#pragma unroll
                for (int m = 0; m < MT; ++m)
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        bool ok;
                        const float* p = ld.ptr(rs[m][i], ks, ok);
                        const int n = ok ? 16 : 0;
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + m * (TC_BM * TC_BK * 4) + aoff[i]), "l"(p), "r"(n) : "memory");
                    }
                // arrive on raw_full[sr] once every cp.async issued so far by this thread has landed
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(raw_full(sr)) : "memory");
            }
        }
        cp_async_wait_all();
    } else if (warp < 8) {
        // ------------------------------------------ A splitters ------------------------------------------
        const int q = warp & 3;                                  // TMEM lane quarter of this warp
        const int r = q * 32 + lane;                             // the row (TMEM lane) owned by this thread
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        uint32_t roff[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) roff[c] = tc_swz(r, c);
        const int64_t total = (int64_t)n_my_units * KBA;
        TcRing rr, ra;
        for (int64_t slot = 0; slot < total; ++slot, rr.next_of(SRn), ra.template next<SA>()) {
            const uint32_t sr = rr.s, pr = rr.ph;
            const uint32_t sa = ra.s, pa = ra.ph;
            bool ok1, ok2;
            ok1 = mbar_wait(raw_full(sr), pr, abort_flag, 5, &g_tc_status);
            if (!ok1) break;
            ok2 = mbar_wait(a_empty(sa), pa ^ 1, abort_flag, 8, &g_tc_status);
            if (!ok2) break;
            tc_fence_after();
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const uint8_t* src = raw + sr * C::RAW_BYTES + m * (TC_BM * TC_BK * 4);
                float4 v[8];
                if constexpr (Loader::COLUMN_SPLIT) {
                    // element k of this thread's row of A is float `lane` of tile row q * 32 + k (consecutive lanes read
                    // consecutive floats of one 128-byte tile row: no bank conflicts)
                    float* vf = reinterpret_cast<float*>(v);
                    // tile row q * 32 + k: byte offset (4 q + k / 8) * 1024 + (k % 8) * 128, chunk (lane / 4) ^ (k % 8): eight
                    // per-thread bases (one per k % 8), everything else is a constant offset of the load
                    const uint8_t* cb[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) cb[j] = src + q * 4096 + j * 128 + (((lane >> 2) ^ j) << 4) + (lane & 3) * 4;
#pragma unroll
                    for (int k = 0; k < 32; ++k) vf[k] = *reinterpret_cast<const float*>(cb[k & 7] + (k >> 3) * 1024);
                }
                const uint32_t a_hi = tmem_a + lane_addr + (sa * MT + m) * 64;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float4 w;
                        if constexpr (Loader::COLUMN_SPLIT) w = v[4 * h + j];
                        else w = *reinterpret_cast<const float4*>(src + roff[4 * h + j]);      // (loaded per half: fewer live registers)
                        split_tf32(w.x, hi[4 * j], lo[4 * j]); split_tf32(w.y, hi[4 * j + 1], lo[4 * j + 1]);
                        split_tf32(w.z, hi[4 * j + 2], lo[4 * j + 2]); split_tf32(w.w, hi[4 * j + 3], lo[4 * j + 3]);
                    }
                    tc_st16(a_hi + 16 * h, hi);
                    tc_st16(a_hi + 32 + 16 * h, lo);
                }
            }
            mbar_arrive(raw_empty(sr));                         // the raw stage has been read
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(a_full(sa));
        }
    } else if (warp == TC_BLOAD_WARP) {
        // ------------------------------------------ W loader ------------------------------------------
        if constexpr (Loader::W_CONVERT) {
            // The whole warp works: lane 0 bulk-copies the prepared image of every k-block but the last; for the last one the
            // unit's plain [rows][32] block is fetched with cp.async into a small ring three units ahead (a global load
            // takes longer than a unit), then lane n splits column n and stores it as row n of the W stage image (k = row of
            // the block; the k padding of the stages is cleared once).
            constexpr int SBR = Loader::W_TAIL_RESIDENT ? SB - 1 : SB;          // stages of the ring
            for (int i = lane; i < SBR * (int)B_STAGE / 16; i += 32)
                reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
            __syncwarp();
            if (Loader::W_TAIL_RESIDENT && lane == 0 && n_my_units > 0) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b_full(SB - 1)), "r"((uint32_t)C::B_BYTES) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_base + (SB - 1) * B_STAGE), "l"(ld.w_src(wtile, 0, 0, C::B_BYTES / 4)),
                               "r"((uint32_t)C::B_BYTES), "r"(b_full(SB - 1)) : "memory");
            }
            const int prow = ld.w_plain_rows();
            float* praw = reinterpret_cast<float*>(bar_mem + C::BAR_BYTES);           // [4][32 rows][32] plain blocks
            auto fetch = [&](int ui_) {
                if (ui_ < n_my_units) {
                    const float* src = ld.w_plain(unit_index(ui_));
                    float* dst = praw + (ui_ & 3) * 1024;
                    for (int i = lane; i < prow * 8; i += 32) cp_async_zfill<16>(dst + 4 * i, src + 4 * i, true);
                }
                cp_async_commit();                              // one group per unit slot, empty past the end
            };
            fetch(0); fetch(1); fetch(2);
            TcRing rb;
            bool alive = true;
            for (int ui = 0; ui < n_my_units && alive; ++ui) {
                cp_async_wait<2>();                             // this unit's block has landed (two younger groups may be in flight)
                __syncwarp();
                if (!mbar_wait(b_empty(rb.s), rb.ph ^ 1, abort_flag, 6, &g_tc_status)) break;
                // lane n writes row n of the image: per 16-byte chunk (four k values) one store of the hi and one of the lo part
                // (this warp's instruction count per unit is on the critical path of the whole pipeline)
                uint8_t* stage = smem + rb.s * B_STAGE;
                const float* blk = praw + (ui & 3) * 1024 + lane;
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    if (4 * c < prow) {
                        uint32_t h[4], l[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float v = (4 * c + e < prow) ? blk[(4 * c + e) * 32] : 0.0f;
                            split_tf32_rn(v, h[e], l[e]);
                        }
                        const uint32_t off = tc_swz(lane, c);
                        *reinterpret_cast<uint4*>(stage + off) = make_uint4(h[0], h[1], h[2], h[3]);
                        *reinterpret_cast<uint4*>(stage + BN * TC_BK * 4 + off) = make_uint4(l[0], l[1], l[2], l[3]);
                    }
                }
                fence_proxy_async();                            // generic-proxy stores before the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(b_full(rb.s));
                rb.template next<SBR>();
                fetch(ui + 3);                                  // into the slot of unit ui - 1, which has been stored
                for (int kb = 0; kb < (Loader::W_TAIL_RESIDENT ? 0 : KB - 1); ++kb, rb.template next<SBR>()) {
                    if (!mbar_wait(b_empty(rb.s), rb.ph ^ 1, abort_flag, 6, &g_tc_status)) { alive = false; break; }
                    if (lane == 0) {
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b_full(rb.s)), "r"((uint32_t)C::B_BYTES) : "memory");
                        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                     ::"r"(smem_base + rb.s * B_STAGE), "l"(ld.w_src(wtile, unit_index(ui), kb, C::B_BYTES / 4)),
                                       "r"((uint32_t)C::B_BYTES), "r"(b_full(rb.s)) : "memory");
                    }
                }
            }
            cp_async_wait_all();
        } else
        if (lane == 0 && n_my_units > 0) {
            const uint32_t bytes = C::B_BYTES;
            const int64_t total = resident ? KB : (int64_t)n_my_units * KB;
            TcRing rb;
            int kbw = 0, uiw = 0;
            for (int64_t slot = 0; slot < total; ++slot, rb.template next<SB>()) {
                const uint32_t sb = rb.s, ph = rb.ph;
                if (!mbar_wait(b_empty(sb), ph ^ 1, abort_flag, 6, &g_tc_status)) break;
                const int kb = kbw;
                const float* wsrc = ld.w_src(wtile, unit_index(uiw), kb, C::B_BYTES / 4);
                if (++kbw == KB) { kbw = 0; ++uiw; }
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b_full(sb)), "r"(bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_base + sb * B_STAGE), "l"(wsrc), "r"(bytes), "r"(b_full(sb)) : "memory");
            }
        }
        __syncwarp();
    } else if (warp < TC_MMA_WARP + NIWARPS) {
        // ------------------------------------------ MMA issuers ------------------------------------------
        // One thread issues a tcgen05.mma about every 54 cycles, while a 128 x 64 x 8 tf32 MMA occupies the tensor
        // pipe for 32 cycles (128 x 128 x 8: 64), so a single issuing thread can starve the pipe.  With two row tiles
        // per unit (MT == 2) two warps issue concurrently, one tile (its own accumulator) each; both wait on the same
        // full barriers and the empty / accumulator barriers expect one commit from each.
        const int iw = warp - TC_MMA_WARP;
        constexpr int NI = BN;                                              // N of one instruction
        {
        constexpr uint32_t idesc = tc_idesc(NI);
        const uint32_t d_off = (MT == 2) ? (uint32_t)(iw * C::ACCW) : (uint32_t)(iw * NI);
        const uint32_t a_off = (MT == 2) ? (uint32_t)(iw * 64) : 0u;
        const uint32_t b_off = (MT == 2) ? 0u : (uint32_t)(iw * NI * 128);   // NI rows of 128 bytes
        // Only lane 0 runs the loop (waits included): no divergence and reconvergence per k-block.  The B descriptors
        // differ between stages only in the address field of their low word, so they are advanced with 32-bit adds.
        {
            const uint32_t leader = lane == 0 ? 1u : 0u;      // the whole warp runs the loop, this lane issues
            const uint64_t desc0 = tc_smem_desc(smem_base + b_off);
            const uint32_t desc_hi = (uint32_t)(desc0 >> 32), desc_lo0 = (uint32_t)desc0;
            TcRing ra, rb;
            bool alive = true;
            for (int ui = 0; ui < n_my_units && alive; ++ui) {
                const uint32_t buf = (uint32_t)(ui % NBUF), aph = (uint32_t)((ui / NBUF) & 1);
                bool okc; okc = mbar_wait(acc_empty(buf), aph ^ 1, abort_flag, 2, &g_tc_status);
                if (!okc) break;
                tc_fence_after();
                const uint32_t d = tmem_base + buf * MT * C::ACCW + d_off;
                for (int ki = 0; ki < KB; ++ki) {
                    // With a constant A block its k-block comes first: it needs no A stage, so its MMAs are issued while
                    // the splitters still work on the unit (the W loader fills the stages in the same order).
                    const int kb = Loader::CONST_A ? (ki == 0 ? KB - 1 : ki - 1) : ki;
                    const uint32_t sa = ra.s, pa = ra.ph;
                    const bool a_ring = kb < KBA;                     // else: the constant A k-block
                    const bool tail = Loader::W_TAIL_RESIDENT && a_ring;   // this k-block's W image stays in the last stage
                    constexpr int SBR = Loader::W_TAIL_RESIDENT ? SB - 1 : SB;
                    const uint32_t sb = resident ? (uint32_t)kb : (tail ? (uint32_t)(SB - 1) : rb.s);
                    bool oka = true, okb = true;
                    if (a_ring) oka = mbar_wait(a_full(sa), pa, abort_flag, 3, &g_tc_status);
                    if (!oka) { alive = false; break; }
                    if ((!resident && !tail) || ui == 0) {
                        okb = mbar_wait(b_full(sb), (resident || tail) ? 0u : rb.ph, abort_flag, 7, &g_tc_status);
                        if (!okb) { alive = false; break; }
                    }
                    tc_fence_after();
                    const uint32_t bh = desc_lo0 + sb * (B_STAGE >> 4), bl = bh + (B_STAGE >> 5);
                    const uint32_t ah = (a_ring ? tmem_a + sa * MT * 64 : tmem_c) + a_off, al = ah + 32;
                    if constexpr (C::MERGE) {
                        constexpr uint32_t idesc2 = tc_idesc(2 * NI);           // [W_hi | W_lo] as one operand of twice the rows
                        const int nk8 = (Loader::CONST_A && !a_ring) ? ld.const_ksteps() : TC_BK / 8;   // (zero k-steps of the constant block are skipped)
                        tc_mma_tf32_ts_p_w(d, ah, bh, desc_hi, idesc2, ki > 0 ? 1u : 0u, leader);
                        tc_mma_tf32_ts_acc_w(d, al, bh, desc_hi, idesc, leader);
#pragma unroll
                        for (int k8 = 1; k8 < TC_BK / 8; ++k8) {
                            if (k8 < nk8) {
                                tc_mma_tf32_ts_acc_w(d, ah + k8 * 8, bh + k8 * 2, desc_hi, idesc2, leader);
                                tc_mma_tf32_ts_acc_w(d, al + k8 * 8, bh + k8 * 2, desc_hi, idesc, leader);
                            }
                        }
                    } else {
                    tc_mma_tf32_ts_p_w(d, al, bh, desc_hi, idesc, ki > 0 ? 1u : 0u, leader);
                    tc_mma_tf32_ts_acc_w(d, ah, bl, desc_hi, idesc, leader);
                    tc_mma_tf32_ts_acc_w(d, ah, bh, desc_hi, idesc, leader);
#pragma unroll
                    for (int k8 = 1; k8 < TC_BK / 8; ++k8) {          // 32 bytes (2 descriptor units) and 8 TMEM columns per k-step
                        tc_mma_tf32_ts_acc_w(d, al + k8 * 8, bh + k8 * 2, desc_hi, idesc, leader);
                        tc_mma_tf32_ts_acc_w(d, ah + k8 * 8, bl + k8 * 2, desc_hi, idesc, leader);
                        tc_mma_tf32_ts_acc_w(d, ah + k8 * 8, bh + k8 * 2, desc_hi, idesc, leader);
                    }
                    }
                    // the A stage (and a streamed W stage) is reusable once every issuer's MMAs have read it
                    if (a_ring) { tc_commit_w(a_empty(sa), leader); ra.template next<SA>(); }
                    if (!resident && !tail) { tc_commit_w(b_empty(sb), leader); rb.template next<SBR>(); }
                }
                if (alive) tc_commit_w(acc_full(buf), leader);
            }
        }
        __syncwarp();
        }
    } else {
        // ------------------------------------------ epilogue ------------------------------------------
        const int q = warp & 3;                                   // TMEM lane quarter this warp may access
        const int ew = warp - TC_EPI_WARP0;
        const int egroup = CS ? 0 : ew >> 3;                      // which units this warp finishes (0 unless two groups alternate)
        const int half = (ew >> 2) & 1;                           // 0 or 1
        const int chalf = CS ? ew >> 3 : 0;                       // column half of the row tile (two groups sharing the units)
        constexpr int UI_STEP = CS ? 1 : EG;
        const int r_in_tile = q * 32 + lane;
        const int mt_e = (MT == 1) ? 0 : half;                    // M-tile served by this thread
        constexpr int CPT = C::CPT;                               // columns served by this thread
        const int col_lo = (MT == 1) ? half * CPT : chalf * CPT;
        const int epi_idx = ew * 32 + lane;
        float* slot_ptr = reinterpret_cast<float*>(staging + epi_idx * C::SLOT_BYTES);
        bool alive = true;
        // LINEAR epilogue with a residual: the residual values of the elements this thread stores in the next store
        // phase are fetched one phase ahead (the first ones while the accumulator is still being computed); a load
        // issued where it is needed queues behind the producers' traffic and stalls the store phase for microseconds.
        constexpr int EP_PASS = C::PASS;
        constexpr int EP_LPR = EP_PASS / 4, EP_RPI = 32 / EP_LPR, EP_NIT = 32 / EP_RPI;
        float4 rres[EP_NIT];
        auto res_fetch = [&](int ui_, int c0_) {
            if constexpr (EPI == EPI_LINEAR && Loader::RESIDUAL) {
                const TcLinearEpi& e = ep;
                const int row0_ = (unit_tile0(ui_) + mt_e) * TC_BM + q * 32 + lane / EP_LPR;
                const int col_ = nt * BN + c0_ + (lane % EP_LPR) * 4;
#pragma unroll
                for (int i = 0; i < EP_NIT; ++i) {
                    const int64_t orow = ld.out_row(row0_ + i * EP_RPI);
                    rres[i] = (col_ < e.N && orow >= 0) ? __ldg(reinterpret_cast<const float4*>(e.residual + orow * e.ldr + col_))
                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
        };
        if constexpr (EPI == EPI_LINEAR && Loader::RESIDUAL) {
            if (ep.residual != nullptr && egroup < n_my_units) res_fetch(egroup, col_lo);
        }
        for (int ui = egroup; ui < n_my_units && alive; ui += UI_STEP) {
            const uint32_t buf = (uint32_t)(ui % NBUF), aph = (uint32_t)((ui / NBUF) & 1);
            float posv[8];                     // PROJ: this row's position values, fetched while the accumulator is still being computed
            if constexpr (EPI == EPI_PROJ) {
                const int prow = (unit_tile0(ui) + mt_e) * TC_BM + r_in_tile;
#pragma unroll
                for (int pp = 0; pp < 8; ++pp)
                    posv[pp] = (pp < ep.d_pos && prow < rows) ? __ldg(ep.pos + (int64_t)prow * ep.d_pos + pp) : 0.0f;
            }
            float head_sc = 0.0f, head_sh = 0.0f;   // HEAD: this row's de-normalisation and frame flag, prepared ahead in the same way
            bool head_edge = false;
            if constexpr (EPI == EPI_HEAD) {
                const int prow = (unit_tile0(ui) + mt_e) * TC_BM + r_in_tile;
                if (half == 0 && prow < rows) {
                    const int prem = prow % (ep.Hh * ep.Ww);
                    head_sc = ep.scale_map ? __ldg(ep.scale_map + prem) : ep.scale;
                    head_sh = ep.shift_map ? __ldg(ep.shift_map + prem) : ep.shift;
                    const int y = prem / ep.Ww, x = prem - y * ep.Ww;
                    head_edge = ep.dirichlet && (y == 0 || x == 0 || y == ep.Hh - 1 || x == ep.Ww - 1);
                }
            }
            bool okf; okf = mbar_wait(acc_full(buf), aph, abort_flag, 4, &g_tc_status);
            if (!okf) { alive = false; break; }
            tc_fence_after();
            const int tile = unit_tile0(ui) + mt_e;
            const int row = tile * TC_BM + r_in_tile;
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (buf * MT + mt_e) * C::ACCW;

            if constexpr (EPI == EPI_LINEAR) {
                const TcLinearEpi& e = ep;
                constexpr int PASS = C::PASS;                    // columns per staging pass
                constexpr int LPR = PASS / 4;                    // lanes per row in the store phase (float4 each)
                constexpr int RPI = 32 / LPR;                    // rows per store instruction
                const uint8_t* warp_stage = staging + ew * 32 * C::SLOT_BYTES;
                const int tile_row0 = tile * TC_BM + q * 32;
                const int64_t out_base = ld.out_row(tile_row0);          // (-1 with out_nvalid <= 0: nothing is stored)
                const int out_nvalid = ld.out_valid(tile_row0);
                // One pass (at most 32 columns per thread): the thread first takes its whole accumulator row into registers
                // and frees the buffer, so the next unit's MMAs start while this one is finished and stored.
                // (with two buffers the early release measured slower, with one and with two epilogue groups: 396 against 378 us
                // for the spectral layer at batch 64)
                constexpr bool EARLY = CPT <= 32 && NBUF == 1;
                float vall[EARLY ? CPT : 16];
                if constexpr (EARLY) {
#pragma unroll
                    for (int cc = 0; cc < CPT; cc += 16) {
                        float v16[16];
                        if constexpr (C::MERGE) tc_ld16_sum(taddr + col_lo + cc, BN, v16); else tc_ld16(taddr + col_lo + cc, v16);
#pragma unroll
                        for (int j = 0; j < 16; ++j) vall[cc + j] = v16[j];
                    }
                    tc_fence_before();
                    mbar_arrive(acc_empty(buf));
                }
                // One accumulator buffer and more columns than fit in registers: the buffer is freed as soon as its last columns
                // have been read.  With 16-column passes the last pass's columns are read one pass early (TAIL2), so the MMAs of
                // the next unit wait for all passes but the last two instead of for all of them.
                constexpr int NP = CPT / PASS;
                constexpr bool TAIL = !EARLY && NBUF == 1 && CS;      // (measured slower on the 48 / 64-wide tiles: 289 against 283 us)
                constexpr bool TAIL2 = TAIL && PASS == 16 && NP >= 2;
                float vlast[TAIL2 ? 16 : 1];
#pragma unroll (EARLY ? CPT / PASS : 1)
                for (int pi = 0; pi < CPT / PASS; ++pi) {
                    const int c0 = col_lo + pi * PASS;
                    // phase 1: each thread finishes its own row (bias, activation) into its padded staging slot
#pragma unroll (EARLY ? 2 : 1)
                    for (int cc = 0; cc < PASS; cc += 16) {
                        float v[16];
                        if constexpr (EARLY) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) v[j] = vall[pi * PASS + cc + j];
                        } else {
                            if (TAIL2 && pi == NP - 1) {
#pragma unroll
                                for (int j = 0; j < 16; ++j) v[j] = vlast[j];
                            } else {
                                if constexpr (C::MERGE) tc_ld16_sum(taddr + c0 + cc, BN, v); else tc_ld16(taddr + c0 + cc, v);
                            }
                            if constexpr (TAIL2) {
                                if (pi == NP - 2) {
                                    if constexpr (C::MERGE) tc_ld16_sum(taddr + c0 + PASS, BN, vlast); else tc_ld16(taddr + c0 + PASS, vlast);
                                    tc_fence_before();
                                    mbar_arrive(acc_empty(buf));
                                }
                            } else if constexpr (TAIL) {
                                if (pi == NP - 1 && cc + 16 >= PASS) { tc_fence_before(); mbar_arrive(acc_empty(buf)); }
                            }
                        }
                        // one branch on the activation per 16 columns, not per element (padding columns beyond N carry a
                        // zero bias and are never stored)
                        auto finish = [&](auto actf) {
#pragma unroll
                            for (int j4 = 0; j4 < 4; ++j4) {
                                const float4 b = *reinterpret_cast<const float4*>(consts + c0 + cc + 4 * j4);
                                *reinterpret_cast<float4*>(slot_ptr + cc + 4 * j4) =
                                    make_float4(actf(v[4 * j4] + b.x), actf(v[4 * j4 + 1] + b.y), actf(v[4 * j4 + 2] + b.z), actf(v[4 * j4 + 3] + b.w));
                            }
                        };
                        if (e.act == SPGT_ACT_SILU2) finish([](float t) { return silu_f(silu_f(t)); });
                        else if (e.act == SPGT_ACT_RELU) finish([](float t) { return fmaxf(t, 0.0f); });
                        else if (e.act == SPGT_ACT_SILU) finish([](float t) { return silu_f(t); });
                        else finish([](float t) { return t; });
                    }
                    __syncwarp();
                    // phase 2: the warp writes its 32 rows with full-line coalesced float4 stores (+ residual)
                    const int col = nt * BN + c0 + (lane % LPR) * 4;
                    static_assert(PASS == EP_PASS && 32 / RPI == EP_NIT, "residual prefetch follows the store phase's mapping");
                    if (col < e.N) {
                        if (Loader::RESIDUAL && e.residual) {
#pragma unroll
                            for (int i = 0; i < 32 / RPI; ++i) {
                                const int rr = i * RPI + lane / LPR;
                                const int64_t orow = ld.out_row(tile_row0 + rr);
                                if (orow >= 0) {
                                    float4 o = *reinterpret_cast<const float4*>(warp_stage + rr * C::SLOT_BYTES + (lane % LPR) * 16);
                                    o.x += rres[i].x; o.y += rres[i].y; o.z += rres[i].z; o.w += rres[i].w;
                                    *reinterpret_cast<float4*>(e.y + orow * e.ldc + col) = o;
                                }
                            }
                        } else {
                            // The 32 GEMM rows of this warp map to consecutive output rows (out_base onwards, the first
                            // out_nvalid of them exist): one address per pass, a constant stride per store.
                            float* yp = e.y + (out_base + lane / LPR) * e.ldc + col;
                            const uint8_t* sp = warp_stage + (lane / LPR) * C::SLOT_BYTES + (lane % LPR) * 16;
#pragma unroll
                            for (int i = 0; i < 32 / RPI; ++i) {
                                if (i * RPI + lane / LPR < out_nvalid)
                                    *reinterpret_cast<float4*>(yp + (int64_t)(i * RPI) * e.ldc) =
                                        *reinterpret_cast<const float4*>(sp + i * RPI * C::SLOT_BYTES);
                            }
                        }
                    }
                    if (Loader::RESIDUAL && e.residual) {                // the next store phase's residual values: next pass, else next unit
                        if (c0 + PASS < col_lo + CPT) res_fetch(ui, c0 + PASS);
                        else if (ui + UI_STEP < n_my_units) res_fetch(ui + UI_STEP, col_lo);
                    }
                    __syncwarp();
                }
            } else if constexpr (EPI == EPI_SPECF) {
                // accumulator lane (x_local = q, c = lane), column j: Y1[image row][j][c]; a warp stores 128 contiguous bytes per j
                static_assert(EPI != EPI_SPECF || (C::MERGE && BN == 32 && MT == 2), "forward y-transform tile shape");
                const TcSpecFwdEpi& e = ep;
                const int64_t img = (int64_t)tile * 4 + q;
#pragma unroll
                for (int cc = 0; cc < 32; cc += 16) {
                    float v[16];
                    tc_ld16_sum(taddr + cc, BN, v);
                    if (img < e.nimg) {
                        float* dst = e.y1 + (img * e.J + cc) * 32 + lane;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (cc + j < e.J) dst[j * 32] = v[j];
                    }
                }
            } else if constexpr (EPI == EPI_PROJ) {
                const TcProjEpi& e = ep;
                const int p = nt;                               // 0: q, 1: k, 2: v
                const int dpk = e.d_pos + 32;
                const bool rok = row < rows;
                const int b = rok ? row / e.S : 0, s_ = rok ? row - b * e.S : 0;
                float* out = e.out[p];
                const float* lnw = e.lnw[p];
#pragma unroll 1
                for (int hd = half; hd < 4; hd += 2) {           // one head = 32 columns = one TMEM load
                    float v[32];
                    tc_ld32(taddr + hd * 32, v);
                    const float4* c4 = reinterpret_cast<const float4*>(consts) + hd * 8;    // bias | LN weight (+32) | LN bias (+64)
#pragma unroll
                    for (int j4 = 0; j4 < 8; ++j4) {
                        const float4 bb = c4[j4];
                        v[4 * j4] += bb.x; v[4 * j4 + 1] += bb.y; v[4 * j4 + 2] += bb.z; v[4 * j4 + 3] += bb.w;
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
                        for (int j4 = 0; j4 < 8; ++j4) {
                            const float4 w = c4[32 + j4], lb = c4[64 + j4];
                            v[4 * j4] = (v[4 * j4] - mu) * inv * w.x + lb.x;
                            v[4 * j4 + 1] = (v[4 * j4 + 1] - mu) * inv * w.y + lb.y;
                            v[4 * j4 + 2] = (v[4 * j4 + 2] - mu) * inv * w.z + lb.z;
                            v[4 * j4 + 3] = (v[4 * j4 + 3] - mu) * inv * w.w + lb.w;
                        }
                    }
                    if (rok) {
                        float* o = out + (((int64_t)b * e.H + hd) * dpk + e.d_pos) * e.S + s_;
#pragma unroll
                        for (int j = 0; j < 32; ++j) o[(int64_t)j * e.S] = v[j];     // lanes = consecutive s: coalesced
#pragma unroll
                        for (int pp = 0; pp < 8; ++pp)
                            if (pp < e.d_pos) out[(((int64_t)b * e.H + hd) * dpk + pp) * e.S + s_] = posv[pp];
                    }
                }
            } else {
                const TcHeadEpi& e = ep;
                // partial row sums of the second column half: one slot per (unit parity within the group, group)
                float* part = reinterpret_cast<float*>(staging) + (((ui / UI_STEP) & 1) * 2 + egroup) * 128;
                const float4* cb = reinterpret_cast<const float4*>(consts);      // b1[128] then w2[128]
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
                if (half == 1) part[r_in_tile] = acc;
                asm volatile("bar.sync %0, %1;" ::"r"(1 + egroup), "n"(32 * TC_EPI_WARPS) : "memory");   // the eight epilogue warps of this group
                if (half == 0 && row < rows) {
                    acc += part[r_in_tile];
                    e.out[row] = head_edge ? 0.0f : (acc + e.b2) * head_sc + head_sh;
                }
            }
            if constexpr (!(EPI == EPI_LINEAR && NBUF == 1 && (CPT <= 32 || CS))) {     // (else the LINEAR epilogue has freed the buffer already)
                tc_fence_before();
                mbar_arrive(acc_empty(buf));
            }
        }
    }
    // teardown: everyone meets, then the allocating warp frees the tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == TC_MMA_WARP) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
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
        const int nt = n / bn, kb = k / TC_BK;
        tc_img_store(img + ((int64_t)nt * KB + kb) * (2 * bn * TC_BK), bn, n % bn, k % TC_BK, v);
    }
}

// Column tile width.  A 128-wide tile keeps W resident in shared memory only up to K = 128; just above that (the
// 136-wide merged attention heads) two 64-wide column tiles with W resident beat one 128-wide tile that re-streams W
// for every row tile, the second read of the rows coming from L2.  At K = 256 the doubled row traffic costs more
// than the W stream (measured: 0.125 vs 0.094 ms for 180k rows).

// 33 - 48 columns with long K (the 42 / 44-channel convs): a 48-wide tile, whose MMAs take three quarters of the time of a
// 64-wide one; only with two row tiles per unit, which is what K > 256 selects below.
static int tc_bn_for(int N, int K) {
    if (N <= 32) return 32;
    if (N <= 48 && K > 256) return 48;
    if (N <= 64) return 64;
    return (K > 128 && K <= 192) ? 64 : 128;
}

template <int BN, int MT, class Loader, int EPI, class EpiParams>
static int tc_launch(Loader ld, const float* wimg, int kpad, int rows, int n_tiles, const EpiParams& ep, cudaStream_t st) {
    static SmemOptIn configured;
    auto kern = tc_gemm_kernel<BN, MT, Loader, EPI, EpiParams>;
    if (int e = smem_opt_in(kern, TcCfg<BN, MT, Loader, EPI>::BYTES, configured)) return e;
    const int m_units = ceil_div(rows, TC_BM * MT);
    int per_nt = num_sms() / n_tiles;                 // CTAs per column tile
    if (per_nt < 1) per_nt = 1;
    if (per_nt > m_units) per_nt = m_units;
    const int grid = per_nt * n_tiles;
    kern<<<grid, tc_threads(MT, tc_epi_groups<Loader, MT, BN, EPI>()), TcCfg<BN, MT, Loader, EPI>::BYTES, st>>>(ld, wimg, kpad, rows, n_tiles, m_units, ep);
    return launch_status();
}

template <class Loader>
static int tc_dispatch_linear(Loader ld, const float* wprep, int K, int N, int rows, const TcLinearEpi& ep, bool long_k, cudaStream_t st) {
    const int bn = tc_bn_for(N, K), kpad = ceil_div(K, TC_BK) * TC_BK, npad = ceil_div(N, bn) * bn;
    const int n_tiles = npad / bn;
    if (long_k && bn == 128) return tc_launch<128, 2, Loader, EPI_LINEAR, TcLinearEpi>(ld, wprep, kpad, rows, n_tiles, ep, st);
    if (long_k && bn == 64) return tc_launch<64, 2, Loader, EPI_LINEAR, TcLinearEpi>(ld, wprep, kpad, rows, n_tiles, ep, st);
    if (long_k && bn == 48) return tc_launch<48, 2, Loader, EPI_LINEAR, TcLinearEpi>(ld, wprep, kpad, rows, n_tiles, ep, st);
    if (bn == 48) return SPGT_ERR_SHAPE;              // (48-wide images are only prepared for K > 256)
    switch (bn) {
        case 32: return tc_launch<32, 1, Loader, EPI_LINEAR, TcLinearEpi>(ld, wprep, kpad, rows, n_tiles, ep, st);
        case 64: return tc_launch<64, 1, Loader, EPI_LINEAR, TcLinearEpi>(ld, wprep, kpad, rows, n_tiles, ep, st);
        default: return tc_launch<128, 1, Loader, EPI_LINEAR, TcLinearEpi>(ld, wprep, kpad, rows, n_tiles, ep, st);
    }
}

// ---- spectral layer: the two y-transforms as tcgen05 GEMMs (called from spectral.cu) ------------------------------
// W image of a [K][N <= 32] matrix (pitch ldw) for 32-wide column tiles: 2 * 32 * ceil(K / 32) * 32 floats.
int spectral_tc_prepare(const float* w_kn, int ldw, int K, int N, float* img, cudaStream_t st) {
    const int kpad = ceil_div(K, TC_BK) * TC_BK;
    tc_weight_prepare_kernel<<<ceil_div(32 * kpad, 256), 256, 0, st>>>(w_kn, ldw, K, N, kpad, 32, 32, img);
    return launch_status();
}
// Y1[image row][j][c] = sum_y F1[j][y] X[image row][y][c] for nimg image rows of r x 32 floats; f1_img = image of F1^T.
int spectral_fwd_y_tc(const float* x, const float* f1_img, float* y1, int r, int J, int64_t nimg, cudaStream_t st) {
    const int64_t units = ceil_div(nimg, (int64_t)8);
    if (units * 256 > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    TcSpecFwd ld;
    ld.x = x; ld.r = r; ld.nimg = nimg; ld.rows = (int)(units * 256); ld.K = r;
    TcSpecFwdEpi ep{y1, J, nimg};
    return tc_launch<32, 2, TcSpecFwd, EPI_SPECF, TcSpecFwdEpi>(ld, f1_img, ceil_div(r, TC_BK) * TC_BK, ld.rows, 1, ep, st);
}
// out[image row][y][o] = act( X[y][:] Wr + F3[y][:] P[image row] + br[o] ); f3 = [upr * 256][32] table, wr_img = W stage image
// of Wr.  r <= 256: p_plain = the P blocks as plain fp32 [image row][J][32]; larger r: p_img = one W stage image (2048
// floats) per image row.
int spectral_inv_y_tc(const float* x, const float* f3, const float* wr_img, const float* p_img, const float* p_plain, int J,
                      const float* br, float* out, int r, int64_t nimg, int act, cudaStream_t st) {
    const int upr = ceil_div(r, 256);
    if (nimg * upr * 256 > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    TcLinearEpi epc{br, nullptr, 0, out, 32, 32, act};
    if (upr == 1) {
        TcSpecInvC ldc;
        ldc.x = x; ldc.f3 = f3; ldc.wr_img = wr_img; ldc.p = p_plain; ldc.J = J; ldc.r = r; ldc.rows = (int)(nimg * 256); ldc.K = 64;
        return tc_launch<32, 2, TcSpecInvC, EPI_LINEAR, TcLinearEpi>(ldc, wr_img, 64, ldc.rows, 1, epc, st);
    }
    TcSpecInv ld;
    ld.x = x; ld.f3 = f3; ld.wr_img = wr_img; ld.p_img = p_img; ld.r = r; ld.upr = upr; ld.rows = (int)(nimg * upr * 256); ld.K = 64;
    TcLinearEpi ep{br, nullptr, 0, out, 32, 32, act};
    return tc_launch<32, 2, TcSpecInv, EPI_LINEAR, TcLinearEpi>(ld, wr_img, 64, ld.rows, 1, ep, st);
}

}  // namespace spgt

using namespace spgt;

extern "C" size_t spgt_tc_weight_bytes(int K, int N) {
    if (K <= 0 || N <= 0) return 0;
    const int bn = tc_bn_for(N, K);
    return (size_t)2 * (ceil_div(N, bn) * bn) * (ceil_div(K, TC_BK) * TC_BK) * sizeof(float);
}

extern "C" int spgt_tc_weight_prepare(const float* w_kn, int ldw, int K, int N, void* out, size_t out_bytes,
                                      spgt_stream_t stream) {
    if (!w_kn || !out) return SPGT_ERR_NULL;
    if (K <= 0 || N <= 0 || ldw < N) return SPGT_ERR_SHAPE;
    if (out_bytes < spgt_tc_weight_bytes(K, N)) return SPGT_ERR_WORKSPACE;
    if (!aligned16(out)) return SPGT_ERR_ALIGN;
    const int bn = tc_bn_for(N, K), kpad = ceil_div(K, TC_BK) * TC_BK, npad = ceil_div(N, bn) * bn;
    tc_weight_prepare_kernel<<<ceil_div(npad * kpad, 256), 256, 0, (cudaStream_t)stream>>>(w_kn, ldw, K, N, kpad, npad, bn,
                                                                                         (float*)out);
    return launch_status();
}


namespace spgt {
int attn_tc_status(); int ffn_tc_status();          // attention_tc.cu, tc_ffn.cu
int attn_tc_status_reset(); int ffn_tc_status_reset();

// One warp waits on a barrier that nobody arrives at, with a limit of `limit_us` microseconds instead of the two
// seconds of the production kernels: the wait gives up, latches `code` in the status word and the kernel returns.
__global__ void tc_wait_expiry_kernel(int code, unsigned long long limit_ns, int* returned) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, code, &g_tc_status, limit_ns);
        *returned = ok ? 1 : 2;
    }
}
}  // namespace spgt

extern "C" int spgt_tc_status(void) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return SPGT_ERR_LAUNCH;
    if (v != 0) return v;
    const int a = spgt::attn_tc_status();
    if (a != 0) return a > 0 ? 100 + a : a;     // 101..109: a wait of the attention kernel gave up
    return spgt::ffn_tc_status();               // 21..33: a wait of the fused feed-forward kernel gave up
}

extern "C" int spgt_tc_status_reset(void) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)) != cudaSuccess) return SPGT_ERR_LAUNCH;
    if (int e = spgt::attn_tc_status_reset()) return e;
    return spgt::ffn_tc_status_reset();
}

extern "C" int spgt_tc_selftest_wait_expiry(int code, int limit_us, int* returned_dev, spgt_stream_t stream) {
    if (!returned_dev) return SPGT_ERR_NULL;
    if (code <= 0 || limit_us <= 0 || limit_us > 100000) return SPGT_ERR_SHAPE;
    tc_wait_expiry_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(code, (unsigned long long)limit_us * 1000ull, returned_dev);
    return launch_status();
}

extern "C" int spgt_linear_tc_fwd(const float* x, int lda, const void* wprep, const float* bias, const float* residual,
                                  int ldr, float* y, int ldc, int rows, int K, int N, int act, spgt_stream_t stream) {
    if (!x || !wprep || !y) return SPGT_ERR_NULL;
    if (rows <= 0 || K <= 0 || N <= 0 || lda < K || ldc < N || (residual && ldr < N)) return SPGT_ERR_SHAPE;
    if ((lda & 3) || (K & 3) || (N & 3) || (ldc & 3) || (residual && (ldr & 3)) || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(wprep) || !aligned16(y) || (residual && !aligned16(residual)) || (bias && !aligned16(bias)))
        return SPGT_ERR_ALIGN;
    TcDense ld;
    ld.x = x; ld.lda = lda; ld.rows = rows; ld.K = K;
    TcLinearEpi ep{bias, residual, ldr, y, ldc, N, act};
    return tc_dispatch_linear(ld, (const float*)wprep, K, N, rows, ep, K > 256, (cudaStream_t)stream);
}

extern "C" int spgt_conv3x3_tc_fwd(const float* x, int cin_pitch, int cin_off, int Cin, const void* wprep, const float* bias,
                                   float* y, int cout_pitch, int cout_off, int Cout, int B, int Hh, int Ww, int act,
                                   spgt_stream_t stream) {
    if (!x || !wprep || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hh <= 0 || Ww <= 0 || Cin <= 0 || Cout <= 0 || cin_off < 0 || cout_off < 0) return SPGT_ERR_SHAPE;
    if (cin_off + Cin > cin_pitch || cout_off + Cout > cout_pitch || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if ((Cin & 3) || (cin_off & 3) || (cin_pitch & 3) || (Cout & 3) || (cout_off & 3) || (cout_pitch & 3)) return SPGT_ERR_SHAPE;
    const int64_t rows64 = (int64_t)B * Hh * Ww;
    if (rows64 > 0x7fffffffLL / 4 || rows64 * cin_pitch > 0x7fffffffLL * 4) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(wprep) || !aligned16(y) || (bias && !aligned16(bias))) return SPGT_ERR_ALIGN;
    TcConv ld;
    ld.x = x; ld.cin_pitch = cin_pitch; ld.cin_off = cin_off; ld.Cin = Cin; ld.Hh = Hh; ld.Ww = Ww; ld.rows = (int)rows64; ld.K = 9 * Cin;
    TcLinearEpi ep{bias, nullptr, 0, y + cout_off, cout_pitch, Cout, act};
    return tc_dispatch_linear(ld, (const float*)wprep, 9 * Cin, Cout, (int)rows64, ep, true, (cudaStream_t)stream);
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
    return tc_launch<128, 1, TcDense, EPI_PROJ, TcProjEpi>(ld, (const float*)wprep_qkv, 128, (int)rows64, 3, ep, (cudaStream_t)stream);
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
    return tc_launch<128, 1, TcDense, EPI_HEAD, TcHeadEpi>(ld, (const float*)w1prep, kpad, (int)rows64, 1, ep, (cudaStream_t)stream);
}
