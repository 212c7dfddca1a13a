// Dense contractions of the hot path on the tensor cores with 3xTF32 (fp32-level accuracy):
//   C[rows, N] = A[rows, K] * W[K, N]   with a pluggable A-tile loader and a fused epilogue.
// A loaders : dense rows (nn.Linear) and implicit-GEMM 3x3 convolution over NHWC (K = 9*Cin).
// Epilogues : bias + activation + residual (row-major store);
//             bias + per-head LayerNorm + head-major transposed store with the position rows (Q/K/V projection);
//             bias + activation + dot with a vector + affine + Dirichlet frame (decoder head).
// CTA tile 128 x BN x 32, 8 warps (4 along rows x 2 along columns), 3-stage cp.async pipeline.
#include "common.cuh"

namespace spgt {

constexpr int G_BM = 128, G_BK = 32, G_AP = 36, G_STAGES = 3, G_THREADS = 256;

// ------------------------------------------------------------------------------------------------------------
// A-tile loaders.  A thread always copies the same k-chunk column for a fixed set of rows ("slots"), so the
// per-row address arithmetic is done once and the per-k arithmetic once per k-tile.
// ------------------------------------------------------------------------------------------------------------
template <int VEC_> struct DenseLoader {
    static constexpr int VEC = VEC_;
    static constexpr int CPR = G_BK / VEC;            // chunks per row
    static constexpr int RPP = G_THREADS / CPR;       // rows per pass
    static constexpr int SLOTS = G_BM / RPP;
    const float* x; int lda; int rows; int K;
    const float* rp[SLOTS]; bool rok[SLOTS]; int kc; bool kok;
    __device__ void init(int row0, int tid) {
        const int r = tid / CPR;
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int row = row0 + r + s * RPP;
            rok[s] = row < rows;
            rp[s] = x + (int64_t)(rok[s] ? row : 0) * lda;
        }
    }
    __device__ void set_k(int k0, int tid) { kc = k0 + (tid % CPR) * VEC; kok = kc < K; if (!kok) kc = 0; }
    __device__ const float* ptr(int s, bool& ok) const { ok = rok[s] && kok; return rp[s] + kc; }
};

template <int VEC_> struct ConvLoader {
    static constexpr int VEC = VEC_;
    static constexpr int CPR = G_BK / VEC;
    static constexpr int RPP = G_THREADS / CPR;
    static constexpr int SLOTS = G_BM / RPP;
    const float* x; int cin_pitch, cin_off, Cin, Hh, Ww; int rows; int K;
    const float* rp[SLOTS]; int py[SLOTS], px[SLOTS];   // py < 0 marks a row outside the problem
    int dy, dx, coff; bool kok;
    __device__ void init(int row0, int tid) {
        const int r = tid / CPR;
#pragma unroll
        for (int s = 0; s < SLOTS; ++s) {
            const int row = row0 + r + s * RPP;
            if (row < rows) {
                const int b = row / (Hh * Ww);
                const int rem = row - b * Hh * Ww;
                py[s] = rem / Ww;
                px[s] = rem - py[s] * Ww;
                rp[s] = x + (int64_t)row * cin_pitch + cin_off;
            } else {
                py[s] = -(1 << 20); px[s] = 0; rp[s] = x;
            }
        }
    }
    __device__ void set_k(int k0, int tid) {
        const int k = k0 + (tid % CPR) * VEC;
        kok = k < K;
        const int tap = kok ? k / Cin : 4;
        const int c = kok ? k - tap * Cin : 0;
        dy = tap / 3 - 1; dx = tap % 3 - 1;
        coff = (dy * Ww + dx) * cin_pitch + c;
    }
    __device__ const float* ptr(int s, bool& ok) const {
        const int yy = py[s] + dy, xx = px[s] + dx;
        ok = kok && yy >= 0 && yy < Hh && xx >= 0 && xx < Ww;
        return ok ? rp[s] + coff : x;
    }
};

// ------------------------------------------------------------------------------------------------------------
// Epilogue parameter blocks
// ------------------------------------------------------------------------------------------------------------
struct LinearEpi {
    const float* bias; const float* residual; int ldr; float* y; int ldc; int act;
};
struct ProjEpi {           // up to three projections (q, k, v) selected by the column-tile group
    const float* w[3]; const float* bias[3]; const float* lnw[3]; const float* lnb[3];
    float* out[3]; float* invsigma[3]; const float* pos;
    float eps; int S, H, d_pos, D;
};
struct HeadEpi {
    const float* b1; const float* w2; float b2, scale, shift; const float* scale_map; const float* shift_map;
    int dirichlet, Hh, Ww, act; float* out;
};

template <int WN> struct GemmSmem {
    static constexpr int BN = 16 * WN;
    static constexpr int BP = BN + 8;
    static constexpr int A_STAGE = G_BM * G_AP;
    static constexpr int B_STAGE = G_BK * BP;
    static constexpr int STAGE = A_STAGE + B_STAGE;
    static constexpr size_t BYTES = (size_t)G_STAGES * STAGE * sizeof(float);
};

// Main loop shared by all variants: accumulates the CTA tile into acc[2][WN][4] per thread.
template <int WN, class Loader>
__device__ __forceinline__ void gemm_mainloop(Loader& ld, const float* __restrict__ W, int ldw, int N, int K, int row0,
                                              int col0, float* smem, float (&acc)[2][WN][4]) {
    using L = GemmSmem<WN>;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int wm = warp >> 1, wn = warp & 1;
    ld.init(row0, tid);
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < WN; ++j)
#pragma unroll
            for (int r = 0; r < 4; ++r) acc[i][j][r] = 0.0f;

    const int KT = (K + G_BK - 1) / G_BK;
    constexpr int B_CPR = L::BN / 4;                        // float4 chunks per B row
    constexpr int B_CHUNKS = G_BK * B_CPR;

    auto load_tile = [&](int kt, int stage) {
        float* as = smem + stage * L::STAGE;
        float* bs = as + L::A_STAGE;
        const int k0 = kt * G_BK;
        ld.set_k(k0, tid);
        const int r = tid / Loader::CPR, kc = (tid % Loader::CPR) * Loader::VEC;
#pragma unroll
        for (int s = 0; s < Loader::SLOTS; ++s) {
            bool ok;
            const float* p = ld.ptr(s, ok);
            cp_async_zfill<Loader::VEC * 4>(as + (r + s * Loader::RPP) * G_AP + kc, p, ok);
        }
        for (int c = tid; c < B_CHUNKS; c += G_THREADS) {
            const int kr = c / B_CPR, nc = (c % B_CPR) * 4;
            const int k = k0 + kr, n = col0 + nc;
            const bool ok = k < K && n < N;
            cp_async_zfill<16>(bs + kr * L::BP + nc, W + (ok ? (int64_t)k * ldw + n : 0), ok);
        }
    };

#pragma unroll
    for (int s = 0; s < G_STAGES - 1; ++s) {
        if (s < KT) load_tile(s, s);
        cp_async_commit();
    }
    for (int kt = 0; kt < KT; ++kt) {
        cp_async_wait<G_STAGES - 2>();
        __syncthreads();
        if (kt + G_STAGES - 1 < KT) load_tile(kt + G_STAGES - 1, (kt + G_STAGES - 1) % G_STAGES);
        cp_async_commit();
        const float* as = smem + (kt % G_STAGES) * L::STAGE;
        const float* bs = as + L::A_STAGE;
#pragma unroll
        for (int k8 = 0; k8 < G_BK / 8; ++k8) {
            const int kk = k8 * 8 + t;
            uint32_t ahi[2][4], alo[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float* p = as + (wm * 32 + i * 16 + g) * G_AP + kk;
                split_tf32(p[0], ahi[i][0], alo[i][0]);
                split_tf32(p[8 * G_AP], ahi[i][1], alo[i][1]);
                split_tf32(p[4], ahi[i][2], alo[i][2]);
                split_tf32(p[8 * G_AP + 4], ahi[i][3], alo[i][3]);
            }
            constexpr int JG = WN < 4 ? WN : 4;          // n-tiles per group: keeps the B fragments in registers
#pragma unroll
            for (int j0 = 0; j0 < WN; j0 += JG) {
                uint32_t bhi[JG][2], blo[JG][2];
#pragma unroll
                for (int j = 0; j < JG; ++j) {
                    if (j0 + j < WN) {
                        const float* p = bs + kk * L::BP + wn * (8 * WN) + (j0 + j) * 8 + g;
                        split_tf32(p[0], bhi[j][0], blo[j][0]);
                        split_tf32(p[4 * L::BP], bhi[j][1], blo[j][1]);
                    }
                }
                // three passes: consecutive MMAs never touch the same accumulator
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < JG; ++j) if (j0 + j < WN) mma_tf32(acc[i][j0 + j], alo[i], bhi[j]);
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < JG; ++j) if (j0 + j < WN) mma_tf32(acc[i][j0 + j], ahi[i], blo[j]);
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < JG; ++j) if (j0 + j < WN) mma_tf32(acc[i][j0 + j], ahi[i], bhi[j]);
            }
        }
    }
    cp_async_wait<0>();
    __syncthreads();      // the pipeline buffers may now be reused by an epilogue
}

// ------------------------------------------------------------------------------------------------------------
// Linear / convolution kernel: y = act(A*W + bias) (+ residual), row-major store.
// ------------------------------------------------------------------------------------------------------------
template <int WN, class Loader>
__global__ void __launch_bounds__(G_THREADS, 2)
gemm_linear_kernel(Loader ld, const float* __restrict__ W, int ldw, int N, int K, int rows, int n_tiles, LinearEpi ep) {
    extern __shared__ __align__(16) float smem[];
    const int row0 = (blockIdx.x / n_tiles) * G_BM;
    const int col0 = (blockIdx.x % n_tiles) * (16 * WN);
    float acc[2][WN][4];
    gemm_mainloop<WN, Loader>(ld, W, ldw, N, K, row0, col0, smem, acc);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3, wm = warp >> 1, wn = warp & 1;
    const bool vec2 = ((ep.ldc & 1) == 0) && ((reinterpret_cast<uintptr_t>(ep.y) & 7) == 0) &&
                      (ep.residual == nullptr || (((ep.ldr & 1) == 0) && ((reinterpret_cast<uintptr_t>(ep.residual) & 7) == 0)));
#pragma unroll
    for (int j = 0; j < WN; ++j) {
        const int col = col0 + wn * (8 * WN) + j * 8 + 2 * t;
        if (col >= N) continue;
        const bool has1 = col + 1 < N;
        const float b0 = ep.bias ? __ldg(ep.bias + col) : 0.0f;
        const float b1 = (ep.bias && has1) ? __ldg(ep.bias + col + 1) : 0.0f;
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int row = row0 + wm * 32 + i * 16 + g + hf * 8;
                if (row >= rows) continue;
                float v0 = apply_act(acc[i][j][2 * hf] + b0, ep.act);
                float v1 = apply_act(acc[i][j][2 * hf + 1] + b1, ep.act);
                float* yp = ep.y + (int64_t)row * ep.ldc + col;
                if (vec2 && has1) {
                    if (ep.residual) {
                        const float2 r = __ldg(reinterpret_cast<const float2*>(ep.residual + (int64_t)row * ep.ldr + col));
                        v0 += r.x; v1 += r.y;
                    }
                    *reinterpret_cast<float2*>(yp) = make_float2(v0, v1);
                } else {
                    if (ep.residual) {
                        v0 += __ldg(ep.residual + (int64_t)row * ep.ldr + col);
                        if (has1) v1 += __ldg(ep.residual + (int64_t)row * ep.ldr + col + 1);
                    }
                    yp[0] = v0;
                    if (has1) yp[1] = v1;
                }
            }
    }
}

// ------------------------------------------------------------------------------------------------------------
// Q/K/V projection kernel: column-tile group p = 0..nproj-1 selects the weight set; 128 columns = 4 heads.
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(G_THREADS, 2)
gemm_proj_kernel(DenseLoader<4> ld, int rows, int nproj, ProjEpi ep) {
    constexpr int WN = 8;
    constexpr int CP = G_BM + 4;                  // staging pitch (column-major tile): == 4 (mod 32)
    extern __shared__ __align__(16) float smem[];
    const int tiles_per_proj = ep.D / 128;
    const int ct = blockIdx.x % (tiles_per_proj * nproj);
    const int p = ct / tiles_per_proj;
    const int col0 = (ct % tiles_per_proj) * 128;
    const int row0 = (blockIdx.x / (tiles_per_proj * nproj)) * G_BM;
    float acc[2][WN][4];
    gemm_mainloop<WN, DenseLoader<4>>(ld, ep.w[p], ep.D, ep.D, ep.D, row0, col0, smem, acc);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3, wm = warp >> 1, wn = warp & 1;
    const float* bias = ep.bias[p];
    const float* lnw = ep.lnw[p];
    const float* lnb = ep.lnb[p];
    float* invs = ep.invsigma[p];
    const int dpk = ep.d_pos + 32;

    // bias, then LayerNorm over each head's 32 columns: a quad (4 lanes with the same g) holds one row of a head
#pragma unroll
    for (int j = 0; j < WN; ++j) {
        const int col = col0 + wn * 64 + j * 8 + 2 * t;
        const float b0 = bias ? __ldg(bias + col) : 0.0f, b1 = bias ? __ldg(bias + col + 1) : 0.0f;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            acc[i][j][0] += b0; acc[i][j][1] += b1; acc[i][j][2] += b0; acc[i][j][3] += b1;
        }
    }
    if (lnw != nullptr) {
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {           // the warp's 64 columns = 2 heads
            const int head = (col0 + wn * 64) / 32 + hh;
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    float s = 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) s += acc[i][hh * 4 + j][2 * hf] + acc[i][hh * 4 + j][2 * hf + 1];
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    const float mu = s * (1.0f / 32.0f);
                    float q = 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float d0 = acc[i][hh * 4 + j][2 * hf] - mu, d1 = acc[i][hh * 4 + j][2 * hf + 1] - mu;
                        q += d0 * d0 + d1 * d1;
                    }
                    q += __shfl_xor_sync(0xffffffffu, q, 1);
                    q += __shfl_xor_sync(0xffffffffu, q, 2);
                    const float inv = 1.0f / sqrtf(q * (1.0f / 32.0f) + ep.eps);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int c = j * 8 + 2 * t;
                        const float w0 = __ldg(lnw + head * 32 + c), w1 = __ldg(lnw + head * 32 + c + 1);
                        const float o0 = __ldg(lnb + head * 32 + c), o1 = __ldg(lnb + head * 32 + c + 1);
                        acc[i][hh * 4 + j][2 * hf] = (acc[i][hh * 4 + j][2 * hf] - mu) * inv * w0 + o0;
                        acc[i][hh * 4 + j][2 * hf + 1] = (acc[i][hh * 4 + j][2 * hf + 1] - mu) * inv * w1 + o1;
                    }
                    if (invs != nullptr && t == 0) {
                        const int row = row0 + wm * 32 + i * 16 + g + hf * 8;
                        if (row < rows) {
                            const int b = row / ep.S, s_ = row - b * ep.S;
                            invs[((int64_t)b * ep.H + head) * ep.S + s_] = inv;
                        }
                    }
                }
        }
    }
    // stage the tile column-major, then write each column as a run of consecutive sequence positions
    float* cs = smem;
#pragma unroll
    for (int j = 0; j < WN; ++j) {
        const int c = wn * 64 + j * 8 + 2 * t;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = wm * 32 + i * 16 + g;
            cs[c * CP + r] = acc[i][j][0];
            cs[(c + 1) * CP + r] = acc[i][j][1];
            cs[c * CP + r + 8] = acc[i][j][2];
            cs[(c + 1) * CP + r + 8] = acc[i][j][3];
        }
    }
    __syncthreads();
    float* out = ep.out[p];
    int64_t rbase[4]; bool rok[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {                  // lane <-> row (4 passes of 32 rows)
        const int row = row0 + q * 32 + lane;
        rok[q] = row < rows;
        const int b = rok[q] ? row / ep.S : 0, s_ = rok[q] ? row - b * ep.S : 0;
        rbase[q] = (int64_t)b * ep.H * dpk * ep.S + s_;
    }
    for (int c = warp; c < 128; c += 8) {
        const int head = (col0 + c) / 32, ch = (col0 + c) % 32;
        const int64_t coff = ((int64_t)head * dpk + ep.d_pos + ch) * ep.S;
#pragma unroll
        for (int q = 0; q < 4; ++q)
            if (rok[q]) out[rbase[q] + coff] = cs[c * CP + q * 32 + lane];
    }
    // position rows of the four heads of this tile
    for (int idx = tid; idx < G_BM * ep.d_pos; idx += G_THREADS) {
        const int r = idx % G_BM, pp = idx / G_BM;
        const int row = row0 + r;
        if (row < rows) {
            const int b = row / ep.S, s_ = row - b * ep.S;
            const float v = __ldg(ep.pos + (int64_t)row * ep.d_pos + pp);
#pragma unroll
            for (int hh = 0; hh < 4; ++hh) {
                const int head = col0 / 32 + hh;
                out[(((int64_t)b * ep.H + head) * dpk + pp) * ep.S + s_] = v;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// Decoder head: out[row] = ((act(A*W1 + b1) . w2) + b2) * scale + shift, zero on the Dirichlet frame.  N1 = 128.
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(G_THREADS, 2)
gemm_head_kernel(DenseLoader<4> ld, const float* __restrict__ W1, int K, int rows, HeadEpi ep) {
    constexpr int WN = 8;
    extern __shared__ __align__(16) float smem[];
    const int row0 = blockIdx.x * G_BM;
    float acc[2][WN][4];
    gemm_mainloop<WN, DenseLoader<4>>(ld, W1, 128, 128, K, row0, 0, smem, acc);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3, wm = warp >> 1, wn = warp & 1;
    float part[2][2] = {{0.0f, 0.0f}, {0.0f, 0.0f}};
#pragma unroll
    for (int j = 0; j < WN; ++j) {
        const int col = wn * 64 + j * 8 + 2 * t;
        const float b0 = __ldg(ep.b1 + col), b1 = __ldg(ep.b1 + col + 1);
        const float w0 = __ldg(ep.w2 + col), w1 = __ldg(ep.w2 + col + 1);
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf)
                part[i][hf] += apply_act(acc[i][j][2 * hf] + b0, ep.act) * w0 + apply_act(acc[i][j][2 * hf + 1] + b1, ep.act) * w1;
    }
    float* red = smem;       // [2][128]
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
            float s = part[i][hf];
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            if (t == 0) red[wn * G_BM + wm * 32 + i * 16 + g + hf * 8] = s;
        }
    __syncthreads();
    if (tid < G_BM) {
        const int row = row0 + tid;
        if (row < rows) {
            const int rem = row % (ep.Hh * ep.Ww);
            const float sc = ep.scale_map ? __ldg(ep.scale_map + rem) : ep.scale;
            const float sh = ep.shift_map ? __ldg(ep.shift_map + rem) : ep.shift;
            float v = (red[tid] + red[G_BM + tid] + ep.b2) * sc + sh;
            if (ep.dirichlet) {
                const int y = rem / ep.Ww, x = rem - y * ep.Ww;
                if (y == 0 || x == 0 || y == ep.Hh - 1 || x == ep.Ww - 1) v = 0.0f;
            }
            ep.out[row] = v;
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// host launchers
// ------------------------------------------------------------------------------------------------------------
template <int WN, class Loader>
static int launch_linear(Loader ld, const float* W, int ldw, int N, int K, int rows, const LinearEpi& ep, cudaStream_t st) {
    static SmemOptIn done;
    auto kern = gemm_linear_kernel<WN, Loader>;
    if (int e = smem_opt_in(kern, GemmSmem<WN>::BYTES, done)) return e;
    const int n_tiles = ceil_div(N, 16 * WN);
    const int64_t blocks = (int64_t)ceil_div(rows, G_BM) * n_tiles;
    if (blocks > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    kern<<<(unsigned)blocks, G_THREADS, GemmSmem<WN>::BYTES, st>>>(ld, W, ldw, N, K, rows, n_tiles, ep);
    return launch_status();
}

template <class Loader>
static int dispatch_linear(Loader ld, const float* W, int ldw, int N, int K, int rows, const LinearEpi& ep, cudaStream_t st) {
    if (N > 64) return launch_linear<8, Loader>(ld, W, ldw, N, K, rows, ep, st);
    if (N > 48) return launch_linear<4, Loader>(ld, W, ldw, N, K, rows, ep, st);
    if (N > 32) return launch_linear<3, Loader>(ld, W, ldw, N, K, rows, ep, st);
    return launch_linear<2, Loader>(ld, W, ldw, N, K, rows, ep, st);
}

}  // namespace spgt

using namespace spgt;

extern "C" int spgt_linear_fwd(const float* x, int lda, const float* w, int ldw, const float* bias, const float* residual,
                               int ldr, float* y, int ldc, int rows, int K, int N, int act, spgt_stream_t stream) {
    if (!x || !w || !y) return SPGT_ERR_NULL;
    if (rows <= 0 || K <= 0 || N <= 0 || lda < K || ldc < N || ldw < N || (residual && ldr < N)) return SPGT_ERR_SHAPE;
    if ((lda & 3) || (K & 3) || (ldw & 3) || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(w) || !aligned16(y)) return SPGT_ERR_ALIGN;
    DenseLoader<4> ld;
    ld.x = x; ld.lda = lda; ld.rows = rows; ld.K = K;
    LinearEpi ep{bias, residual, ldr, y, ldc, act};
    return dispatch_linear(ld, w, ldw, N, K, rows, ep, (cudaStream_t)stream);
}

extern "C" int spgt_conv3x3_fwd(const float* x, int cin_pitch, int cin_off, int Cin, const float* w, int ldw,
                                const float* bias, float* y, int cout_pitch, int cout_off, int Cout, int B, int Hh, int Ww,
                                int act, spgt_stream_t stream) {
    if (!x || !w || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hh <= 0 || Ww <= 0 || Cin <= 0 || Cout <= 0 || cin_off < 0 || cout_off < 0) return SPGT_ERR_SHAPE;
    if (cin_off + Cin > cin_pitch || cout_off + Cout > cout_pitch || ldw < Cout || (ldw & 3) || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if ((Cin & 1) || (cin_off & 1) || (cin_pitch & 1)) return SPGT_ERR_SHAPE;
    const int64_t rows64 = (int64_t)B * Hh * Ww;
    if (rows64 > 0x7fffffffLL / 4 || rows64 * cin_pitch > 0x7fffffffLL * 4) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(w) || !aligned16(y)) return SPGT_ERR_ALIGN;
    const int rows = (int)rows64;
    LinearEpi ep{bias, nullptr, 0, y + cout_off, cout_pitch, act};
    cudaStream_t st = (cudaStream_t)stream;
    if ((Cin & 3) == 0 && (cin_off & 3) == 0 && (cin_pitch & 3) == 0) {
        ConvLoader<4> ld;
        ld.x = x; ld.cin_pitch = cin_pitch; ld.cin_off = cin_off; ld.Cin = Cin; ld.Hh = Hh; ld.Ww = Ww; ld.rows = rows; ld.K = 9 * Cin;
        return dispatch_linear(ld, w, ldw, Cout, 9 * Cin, rows, ep, st);
    }
    ConvLoader<2> ld;
    ld.x = x; ld.cin_pitch = cin_pitch; ld.cin_off = cin_off; ld.Cin = Cin; ld.Hh = Hh; ld.Ww = Ww; ld.rows = rows; ld.K = 9 * Cin;
    return dispatch_linear(ld, w, ldw, Cout, 9 * Cin, rows, ep, st);
}

static int proj_common(const float* x, int nproj, ProjEpi& ep, int B, int S, int D, int H, int d_head, int d_pos,
                       cudaStream_t st) {
    if (B <= 0 || S <= 0 || D <= 0 || H <= 0) return SPGT_ERR_SHAPE;
    if (d_head != 32 || D != H * d_head || (D % 128) != 0 || d_pos < 0 || d_pos > 8) return SPGT_ERR_SHAPE;
    const int64_t rows64 = (int64_t)B * S;
    if (rows64 > 0x7fffffffLL / 2) return SPGT_ERR_SHAPE;
    if (d_pos > 0 && !ep.pos) return SPGT_ERR_NULL;
    static SmemOptIn done;
    if (int e = smem_opt_in(gemm_proj_kernel, GemmSmem<8>::BYTES, done)) return e;
    static_assert(GemmSmem<8>::BYTES >= (size_t)128 * (G_BM + 4) * sizeof(float), "staging tile must fit");
    DenseLoader<4> ld;
    ld.x = x; ld.lda = D; ld.rows = (int)rows64; ld.K = D;
    ep.S = S; ep.H = H; ep.d_pos = d_pos; ep.D = D;
    const int64_t blocks = (int64_t)ceil_div((int)rows64, G_BM) * (D / 128) * nproj;
    if (blocks > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    gemm_proj_kernel<<<(unsigned)blocks, G_THREADS, GemmSmem<8>::BYTES, st>>>(ld, (int)rows64, nproj, ep);
    return launch_status();
}

extern "C" int spgt_projpos_fwd(const float* x, const float* w, const float* bias, const float* pos, float* out, int B,
                                int S, int D, int H, int d_head, int d_pos, spgt_stream_t stream) {
    if (!x || !w || !out) return SPGT_ERR_NULL;
    if (!aligned16(x) || !aligned16(w) || !aligned16(out)) return SPGT_ERR_ALIGN;
    ProjEpi ep = {};
    ep.w[0] = w; ep.bias[0] = bias; ep.out[0] = out; ep.pos = pos; ep.eps = 0.0f;
    return proj_common(x, 1, ep, B, S, D, H, d_head, d_pos, (cudaStream_t)stream);
}

extern "C" int spgt_projpos_lnorm_fwd(const float* x, const float* w, const float* bias, const float* lnw,
                                      const float* lnb, float eps, const float* pos, float* out, float* invsigma, int B,
                                      int S, int D, int H, int d_head, int d_pos, spgt_stream_t stream) {
    if (!x || !w || !out || !lnw || !lnb) return SPGT_ERR_NULL;
    if (!aligned16(x) || !aligned16(w) || !aligned16(out)) return SPGT_ERR_ALIGN;
    ProjEpi ep = {};
    ep.w[0] = w; ep.bias[0] = bias; ep.lnw[0] = lnw; ep.lnb[0] = lnb; ep.out[0] = out; ep.invsigma[0] = invsigma;
    ep.pos = pos; ep.eps = eps;
    return proj_common(x, 1, ep, B, S, D, H, d_head, d_pos, (cudaStream_t)stream);
}

extern "C" int spgt_projpos_qkv_fwd(const float* x, const float* wq, const float* bq, const float* wk, const float* bk,
                                    const float* wv, const float* bv, const float* lnwk, const float* lnbk,
                                    const float* lnwv, const float* lnbv, float eps, const float* pos, float* q,
                                    float* k, float* v, int B, int S, int D, int H, int d_head, int d_pos,
                                    spgt_stream_t stream) {
    if (!x || !wq || !wk || !wv || !q || !k || !v || !lnwk || !lnbk || !lnwv || !lnbv) return SPGT_ERR_NULL;
    if (!aligned16(x) || !aligned16(wq) || !aligned16(wk) || !aligned16(wv) || !aligned16(q) || !aligned16(k) || !aligned16(v))
        return SPGT_ERR_ALIGN;
    ProjEpi ep = {};
    ep.w[0] = wq; ep.bias[0] = bq; ep.out[0] = q;
    ep.w[1] = wk; ep.bias[1] = bk; ep.lnw[1] = lnwk; ep.lnb[1] = lnbk; ep.out[1] = k;
    ep.w[2] = wv; ep.bias[2] = bv; ep.lnw[2] = lnwv; ep.lnb[2] = lnbv; ep.out[2] = v;
    ep.pos = pos; ep.eps = eps;
    return proj_common(x, 3, ep, B, S, D, H, d_head, d_pos, (cudaStream_t)stream);
}

extern "C" int spgt_decoder_head_fwd(const float* x, const float* w1, const float* b1, const float* w2, float b2,
                                     float scale, float shift, const float* scale_map, const float* shift_map,
                                     int dirichlet, float* out, int B, int Hh, int Ww, int K, int N1, int act,
                                     spgt_stream_t stream) {
    if (!x || !w1 || !b1 || !w2 || !out) return SPGT_ERR_NULL;
    if (B <= 0 || Hh <= 0 || Ww <= 0 || K <= 0 || (K & 3) || K > 64 || N1 != 128 || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    const int64_t rows64 = (int64_t)B * Hh * Ww;
    if (rows64 > 0x7fffffffLL / 2) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(w1)) return SPGT_ERR_ALIGN;
    static SmemOptIn done;
    if (int e = smem_opt_in(gemm_head_kernel, GemmSmem<8>::BYTES, done)) return e;
    DenseLoader<4> ld;
    ld.x = x; ld.lda = K; ld.rows = (int)rows64; ld.K = K;
    HeadEpi ep{b1, w2, b2, scale, shift, scale_map, shift_map, dirichlet, Hh, Ww, act, out};
    gemm_head_kernel<<<(unsigned)ceil_div((int)rows64, G_BM), G_THREADS, GemmSmem<8>::BYTES, (cudaStream_t)stream>>>(
        ld, w1, K, (int)rows64, ep);
    return launch_status();
}
