// FNO2d spectral layer as a mode-truncated DFT.
//
// The reference computes rfft2 over the full r x (r/2+1) spectrum, keeps two m x m corner blocks, mixes channels
// per mode, scatters into a zero spectrum and runs irfft2.  Only 2m x m modes are ever non-zero, so the same
// result is obtained from four small contractions (r may be prime, no FFT factorisation is needed):
//   S1  Y1[b,x,j,c]  = sum_y F1[j,y] X[b,x,y,c]          forward DFT along y, j = (re|im) x ky     [tensor cores]
//   S2a Z[b,q,ky,c]  = sum_x G[q,x] Y1c[b,x,ky,c]        forward DFT along x, q = the 2m kept kx   [FFMA]
//   S2b O[b,q,ky,o]  = sum_i Z[b,q,ky,i] W[q,ky,i,o]     complex channel mixing per mode           [FFMA]
//   S2c P[b,x,j,o]   = sum_q conj(G)[q,x] O[b,q,ky,o]    inverse DFT along x                        [FFMA]
//   S3  out[b,x,y,o] = act( sum_j F3[y,j] P[b,x,j,o] + sum_i X[b,x,y,i] Wr[i,o] + br[o] )           [tensor cores]
// F3 carries the Hermitian-symmetry weights of the real inverse transform (1 for ky = 0, 2 otherwise; the
// imaginary part of the ky = 0 column is ignored exactly as a c2r transform does) and both 1/r normalisations
// of norm='ortho' are folded into F1 and F3.  S1 reads X once, S3 reads X once and writes the output once.
#include "common.cuh"

namespace spgt {

constexpr int SP_C = 32;         // channel width handled by the tensor-core kernels
constexpr int SP_WARPS = 4;
constexpr int SP_YB = 32;        // y rows per staged chunk
// pitch of the F1T rows (j): the smallest value >= JP that is 8 or 24 (mod 32), so B-fragment loads are conflict-free
__host__ __device__ constexpr int sp_f1p(int jp) { return jp <= 8 ? 8 : (jp <= 24 ? 24 : 40); }
constexpr int SP_XP1 = 40;       // S1: X chunk pitch (A operand read M-contiguous), == 8 (mod 32)
constexpr int SP_XP3 = 36;       // S3: X chunk pitch (A operand read K-contiguous), == 4 (mod 32)
constexpr int SP_PP = 40;        // S3: P row-block pitch and Wr pitch (B operands), == 8 (mod 32)

constexpr int SP_XMAX = 256;      // largest r the staged S2a / S2c kernels accept (shared-memory budget)
__host__ __device__ inline int sp_round_pitch(int n, int rem) {   // smallest p >= n with p % 32 == rem
    int p = (n + 31) / 32 * 32 + rem;
    if (p - 32 >= n) p -= 32;
    return p;
}

struct SpecTables {              // offsets in floats into the table buffer
    int r, m, J, JP, RY, F3P, F1P;
    int f1t, f3, gr, gi, total;
    int GA_ROWS, GA_P, ga, GC_ROWS, GC_P, gc;    // zero-padded copies of G in the shared-memory layouts of S2a / S2c (r <= SP_XMAX)
};
__host__ __device__ inline SpecTables spec_tables(int r, int m) {
    SpecTables t;
    t.r = r; t.m = m; t.J = 2 * m; t.JP = (2 * m + 7) / 8 * 8; t.RY = (r + SP_YB - 1) / SP_YB * SP_YB; t.F3P = t.JP + 4;
    t.F1P = sp_f1p(t.JP);
    t.f1t = 0;
    t.f3 = t.f1t + t.RY * t.F1P;
    t.gr = t.f3 + t.RY * t.F3P;
    t.gi = t.gr + t.J * r;
    t.total = (t.gi + t.J * r + 3) / 4 * 4;
    t.GA_ROWS = (2 * t.J + 15) / 16 * 16; t.GA_P = sp_round_pitch((r + 7) / 8 * 8, 4);
    t.GC_ROWS = (2 * t.J + 7) / 8 * 8;    t.GC_P = sp_round_pitch((r + 15) / 16 * 16, 8);
    t.ga = t.total; t.gc = t.ga;
    if (r <= SP_XMAX) {
        t.gc = t.ga + t.GA_ROWS * t.GA_P;
        t.total = t.gc + t.GC_ROWS * t.GC_P;
    }
    return t;
}

__device__ __forceinline__ int kept_kx(int q, int r, int m) { return q < m ? q : r - 2 * m + q; }

__global__ void spectral_tables_kernel(float* tab, int r, int m) {
    const SpecTables T = spec_tables(r, m);
    const int n = T.total;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float v = 0.0f;
        if (i < T.f3) {                                        // F1T[y][j]
            const int y = i / T.F1P, j = i % T.F1P;
            if (y < r && j < T.J) {
                const int ky = j < m ? j : j - m;
                double s, c;
                sincospi(2.0 * (double)(((int64_t)ky * y) % r) / (double)r, &s, &c);
                v = (float)((j < m ? c : -s) / (double)r);
            }
        } else if (i < T.gr) {                                 // F3[y][j]
            const int k = i - T.f3;
            const int y = k / T.F3P, j = k % T.F3P;
            if (y < r && j < T.J) {
                const int ky = j < m ? j : j - m;
                const double w = ky == 0 ? 1.0 : 2.0;
                double s, c;
                sincospi(2.0 * (double)(((int64_t)ky * y) % r) / (double)r, &s, &c);
                v = (float)((j < m ? w * c : -w * s) / (double)r);
            }
        } else if (i < T.gi + T.J * r) {                        // G[q][x] = exp(-2 pi i kx_q x / r)
            const bool im = i >= T.gi;
            const int k = i - (im ? T.gi : T.gr);
            const int q = k / r, x = k % r;
            double s, c;
            sincospi(2.0 * (double)(((int64_t)kept_kx(q, r, m) * x) % r) / (double)r, &s, &c);
            v = (float)(im ? -s : c);
        } else if (i >= T.ga && r <= SP_XMAX) {                 // padded copies [rows][pitch]: row q' < 2J = (Re | Im) of G
            const bool c_copy = i >= T.gc;
            const int k = i - (c_copy ? T.gc : T.ga), P = c_copy ? T.GC_P : T.GA_P;
            const int q2 = k / P, x = k % P;
            if (q2 < 2 * T.J && x < r) {
                const int q = q2 < T.J ? q2 : q2 - T.J;
                double s, c;
                sincospi(2.0 * (double)(((int64_t)kept_kx(q, r, m) * x) % r) / (double)r, &s, &c);
                v = (float)(q2 < T.J ? c : -s);
            }
        }
        tab[i] = v;
    }
}

// ------------------------------------------------------------------------------------------------------------
// S1: per (b,x) row  D[c][j] = sum_y X[y][c] * F1T[y][j].   M = c (32), N = j (8*NT), K = y.
// One warp per row at a time; y is streamed in chunks of 32 rows through a private double buffer.
// ------------------------------------------------------------------------------------------------------------
template <int NT>
__global__ void __launch_bounds__(SP_WARPS * 32, 3)
spectral_fwd_y_kernel(const float* __restrict__ X, const float* __restrict__ tab, float* __restrict__ Y1, int r, int m,
                      int64_t nrows) {
    extern __shared__ __align__(16) float smem[];
    const SpecTables T = spec_tables(r, m);
    float* f1 = smem;                                           // [RY][40]
    constexpr int F1P = sp_f1p(8 * NT);
    float* wbuf = smem + T.RY * F1P + (threadIdx.x >> 5) * (2 * SP_YB * SP_XP1);
    for (int i = threadIdx.x; i < T.RY * F1P; i += blockDim.x) f1[i] = __ldg(tab + T.f1t + i);
    __syncthreads();

    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int nchunk = T.RY / SP_YB;
    const int64_t gw = (int64_t)blockIdx.x * SP_WARPS + (threadIdx.x >> 5);
    const int64_t nw = (int64_t)gridDim.x * SP_WARPS;
    const int64_t my_rows = gw < nrows ? (nrows - gw + nw - 1) / nw : 0;
    const int64_t nitem = my_rows * nchunk;

    auto load = [&](int64_t item, int stage) {
        const int64_t row = gw + (item / nchunk) * nw;
        const int y0 = (int)(item % nchunk) * SP_YB;
        const float* src = X + row * (int64_t)r * SP_C;
        float* dst = wbuf + stage * SP_YB * SP_XP1;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int yy = i * 4 + (lane >> 3), c4 = (lane & 7) * 4;
            const bool ok = y0 + yy < r;
            cp_async_zfill<16>(dst + yy * SP_XP1 + c4, src + (int64_t)(ok ? y0 + yy : 0) * SP_C + c4, ok);
        }
        cp_async_commit();
    };

    float acc[2][NT][4];
    if (nitem > 0) load(0, 0);
    for (int64_t it = 0; it < nitem; ++it) {
        if (it + 1 < nitem) { load(it + 1, (int)((it + 1) & 1)); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncwarp();
        const int chunk = (int)(it % nchunk);
        if (chunk == 0) {
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j)
#pragma unroll
                    for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.0f;
        }
        const float* xs = wbuf + (it & 1) * SP_YB * SP_XP1;
        const float* fs = f1 + chunk * SP_YB * F1P;
#pragma unroll
        for (int k8 = 0; k8 < SP_YB / 8; ++k8) {
            const int kk = k8 * 8 + t;
            uint32_t ahi[2][4], alo[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float* p = xs + kk * SP_XP1 + 16 * i + g;        // A[m=c][k=y] = xs[y][c]
                split_tf32(p[0], ahi[i][0], alo[i][0]);
                split_tf32(p[8], ahi[i][1], alo[i][1]);
                split_tf32(p[4 * SP_XP1], ahi[i][2], alo[i][2]);
                split_tf32(p[4 * SP_XP1 + 8], ahi[i][3], alo[i][3]);
            }
            uint32_t bhi[NT][2], blo[NT][2];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const float* p = fs + kk * F1P + 8 * j + g;             // B[k=y][n=j]
                split_tf32(p[0], bhi[j][0], blo[j][0]);
                split_tf32(p[4 * F1P], bhi[j][1], blo[j][1]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_tf32(acc[i][j], alo[i], bhi[j]);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_tf32(acc[i][j], ahi[i], blo[j]);
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_tf32(acc[i][j], ahi[i], bhi[j]);
        }
        __syncwarp();
        if (chunk == nchunk - 1) {
            const int64_t row = gw + (it / nchunk) * nw;
            float* dst = Y1 + row * (int64_t)T.J * SP_C;               // [J][32]
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) {
                    const int c = 16 * i + g, jj = 8 * j + 2 * t;
                    if (jj < T.J) { dst[jj * SP_C + c] = acc[i][j][0]; dst[jj * SP_C + c + 8] = acc[i][j][2]; }
                    if (jj + 1 < T.J) { dst[(jj + 1) * SP_C + c] = acc[i][j][1]; dst[(jj + 1) * SP_C + c + 8] = acc[i][j][3]; }
                }
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// S2a: Z[b,q,ky,c] = sum_x G[q,x] * (Y1[b,x,ky,c] + i Y1[b,x,m+ky,c]).   grid (m, B), lane = c, warp = q stride 8.
// ------------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
spectral_fwd_x_kernel(const float* __restrict__ Y1, const float* __restrict__ tab, float* __restrict__ Zr,
                      float* __restrict__ Zi, int r, int m) {
    extern __shared__ __align__(16) float smem[];
    const SpecTables T = spec_tables(r, m);
    float* gr = smem; float* gi = smem + T.J * r;
    for (int i = threadIdx.x; i < 2 * T.J * r; i += blockDim.x) smem[i] = __ldg(tab + T.gr + i);
    __syncthreads();
    const int ky = blockIdx.x; const int64_t b = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float zr[4] = {0, 0, 0, 0}, zi[4] = {0, 0, 0, 0};
    const float* yb = Y1 + b * (int64_t)r * T.J * SP_C + lane;
#pragma unroll 8
    for (int x = 0; x < r; ++x) {
        const float yr = __ldg(yb + ((int64_t)x * T.J + ky) * SP_C);
        const float yi = __ldg(yb + ((int64_t)x * T.J + m + ky) * SP_C);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int q = warp + 8 * k;
            if (q < T.J) {
                const float a = gr[q * r + x], bb = gi[q * r + x];
                zr[k] = fmaf(a, yr, fmaf(-bb, yi, zr[k]));
                zi[k] = fmaf(a, yi, fmaf(bb, yr, zi[k]));
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int q = warp + 8 * k;
        if (q < T.J) {
            const int64_t o = ((b * T.J + q) * m + ky) * SP_C + lane;
            Zr[o] = zr[k]; Zi[o] = zi[k];
        }
    }
}

// S2b: O[b,q,ky,o] = sum_i Z[b,q,ky,i] * W[q,ky,i,o].   grid = J*m modes, lane = o, warp = b stride 8.
__global__ void __launch_bounds__(256)
spectral_mix_kernel(const float* __restrict__ Zr, const float* __restrict__ Zi, const float* __restrict__ fw0,
                    const float* __restrict__ fw1, float* __restrict__ Or, float* __restrict__ Oi, int B, int m) {
    __shared__ float2 w[SP_C * SP_C];
    const int q = blockIdx.x / m, ky = blockIdx.x % m;
    const float2* src = reinterpret_cast<const float2*>(q < m ? fw0 : fw1) + ((int64_t)(q < m ? q : q - m) * m + ky) * SP_C * SP_C;
    for (int i = threadIdx.x; i < SP_C * SP_C; i += blockDim.x) w[i] = __ldg(src + i);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int J = 2 * m;
    for (int b = warp; b < B; b += 8) {
        const int64_t base = (((int64_t)b * J + q) * m + ky) * SP_C;
        const float zr = __ldg(Zr + base + lane), zi = __ldg(Zi + base + lane);
        float orr = 0.0f, oii = 0.0f;
#pragma unroll
        for (int i = 0; i < SP_C; ++i) {
            const float a = __shfl_sync(0xffffffffu, zr, i), bb = __shfl_sync(0xffffffffu, zi, i);
            const float2 ww = w[i * SP_C + lane];
            orr = fmaf(a, ww.x, fmaf(-bb, ww.y, orr));
            oii = fmaf(a, ww.y, fmaf(bb, ww.x, oii));
        }
        Or[base + lane] = orr; Oi[base + lane] = oii;
    }
}

// S2c: P[b,x,ky,o] + i P[b,x,m+ky,o] = sum_q conj(G[q,x]) * O[b,q,ky,o].   grid (m, B), lane = o, warp = x stride 8.
__global__ void __launch_bounds__(256)
spectral_inv_x_kernel(const float* __restrict__ Or, const float* __restrict__ Oi, const float* __restrict__ tab,
                      float* __restrict__ P, int r, int m) {
    extern __shared__ __align__(16) float smem[];
    const SpecTables T = spec_tables(r, m);
    float* gr = smem; float* gi = smem + T.J * r;
    for (int i = threadIdx.x; i < 2 * T.J * r; i += blockDim.x) smem[i] = __ldg(tab + T.gr + i);
    __syncthreads();
    const int ky = blockIdx.x; const int64_t b = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float orr[32], oii[32];
#pragma unroll
    for (int q = 0; q < 32; ++q) {
        if (q < T.J) {
            const int64_t o = ((b * T.J + q) * m + ky) * SP_C + lane;
            orr[q] = __ldg(Or + o); oii[q] = __ldg(Oi + o);
        } else { orr[q] = 0.0f; oii[q] = 0.0f; }
    }
    for (int x = warp; x < r; x += 8) {
        float pr = 0.0f, pi = 0.0f;
#pragma unroll
        for (int q = 0; q < 32; ++q) {
            if (q < T.J) {
                const float a = gr[q * r + x], bb = gi[q * r + x];     // conj(G) = a - i bb
                pr = fmaf(a, orr[q], fmaf(bb, oii[q], pr));
                pi = fmaf(a, oii[q], fmaf(-bb, orr[q], pi));
            }
        }
        float* dst = P + ((b * r + x) * (int64_t)T.J) * SP_C + lane;
        dst[(int64_t)ky * SP_C] = pr;
        dst[(int64_t)(m + ky) * SP_C] = pi;
    }
}

// ------------------------------------------------------------------------------------------------------------
// S2a and S2c on the tensor cores (3xTF32 warp MMA), one CTA per (ky, b), for r <= SP_XMAX.
//
// S2a as a real GEMM:  R[q'][n] = sum_x Gt[q'][x] * Y[x][n],  q' < 2J (rows 0..J-1 = Re G, J..2J-1 = Im G),
//                      n < 64 (0..31 = Re Y1 = Y1[.., ky, c], 32..63 = Im Y1 = Y1[.., m + ky, c]);
//                      Zr[q][c] = R[q][c] - R[J+q][32+c],  Zi[q][c] = R[q][32+c] + R[J+q][c].
// S2c as a real GEMM:  P[x][n] = sum_k Gt[k][x] * Bm[k][n],  k < 2J,
//                      Bm[q] = (Or[q] | Oi[q]),  Bm[J+q] = (Oi[q] | -Or[q]);  n < 32 -> P[.., ky, :], else P[.., m + ky, :].
// Both stage the whole G table ([2J][r], zero padded) and their Y1 / O block in shared memory, then every warp
// owns a slice of the output (S2a: 16 columns, S2c: every fourth 16-row tile).
// ------------------------------------------------------------------------------------------------------------
constexpr int SP_YP = 72;         // pitch of the [x][64] / [k][64] B operands, == 8 (mod 32)


__global__ void __launch_bounds__(128)
spectral_fwd_x_mma_kernel(const float* __restrict__ Y1, const float* __restrict__ tab, float* __restrict__ Zr,
                          float* __restrict__ Zi, int r, int m) {
    extern __shared__ __align__(16) float smem[];
    const SpecTables T = spec_tables(r, m);
    const int J = T.J, M2 = 2 * J, MT = (M2 + 15) / 16;
    const int r8 = (r + 7) / 8 * 8;
    const int GP = sp_round_pitch(r8, 4);                    // G pitch == 4 (mod 32): A fragments conflict-free
    float* gs = smem;                                        // [16*MT][GP]
    float* ys = smem + 16 * MT * GP;                         // [r8][SP_YP]; later R [16*MT][SP_YP]
    const int ky = blockIdx.x; const int64_t b = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    // Y block: 16 float4 per x (8 from the real row, 8 from the imaginary row)
    const float* yb = Y1 + b * (int64_t)r * J * SP_C;
    for (int i = tid; i < r8 * 16; i += 128) {
        const int x = i >> 4, c4 = i & 15;
        const bool ok = x < r;
        const float* src = yb + ((int64_t)(ok ? x : 0) * J + (c4 < 8 ? ky : m + ky)) * SP_C + (c4 & 7) * 4;
        cp_async_zfill<16>(ys + x * SP_YP + c4 * 4, src, ok);
    }
    cp_async_commit();
    for (int i = tid; i < 16 * MT * GP / 4; i += 128) cp_async_zfill<16>(gs + 4 * i, tab + T.ga + 4 * i, true);   // padded G, as stored
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    float acc[4][2][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;
    const int n0 = warp * 16;
    for (int k0 = 0; k0 < r8; k0 += 8) {
        uint32_t bhi[2][2], blo[2][2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float* p = ys + (k0 + t) * SP_YP + n0 + 8 * j + g;
            split_tf32(p[0], bhi[j][0], blo[j][0]);
            split_tf32(p[4 * SP_YP], bhi[j][1], blo[j][1]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (i < MT) {
                const float* p = gs + (16 * i + g) * GP + k0 + t;
                uint32_t ahi[4], alo[4];
                split_tf32(p[0], ahi[0], alo[0]);
                split_tf32(p[8 * GP], ahi[1], alo[1]);
                split_tf32(p[4], ahi[2], alo[2]);
                split_tf32(p[8 * GP + 4], ahi[3], alo[3]);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    mma_tf32(acc[i][j], alo, bhi[j]);
                    mma_tf32(acc[i][j], ahi, blo[j]);
                    mma_tf32(acc[i][j], ahi, bhi[j]);
                }
            }
        }
    }
    __syncthreads();                                         // everyone is done reading ys
    float* rs = ys;                                          // R [16*MT][SP_YP]
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (i < MT) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int row = 16 * i + g, col = n0 + 8 * j + 2 * t;
                *reinterpret_cast<float2*>(rs + row * SP_YP + col) = make_float2(acc[i][j][0], acc[i][j][1]);
                *reinterpret_cast<float2*>(rs + (row + 8) * SP_YP + col) = make_float2(acc[i][j][2], acc[i][j][3]);
            }
        }
    __syncthreads();
    for (int e = tid; e < J * SP_C; e += 128) {
        const int q = e >> 5, c = e & 31;
        const int64_t o = ((b * J + q) * m + ky) * SP_C + c;
        Zr[o] = rs[q * SP_YP + c] - rs[(J + q) * SP_YP + 32 + c];
        Zi[o] = rs[q * SP_YP + 32 + c] + rs[(J + q) * SP_YP + c];
    }
}

__global__ void __launch_bounds__(128)
spectral_inv_x_mma_kernel(const float* __restrict__ Or, const float* __restrict__ Oi, const float* __restrict__ tab,
                          float* __restrict__ P, int r, int m) {
    extern __shared__ __align__(16) float smem[];
    const SpecTables T = spec_tables(r, m);
    const int J = T.J, M2 = 2 * J, K8 = (M2 + 7) / 8 * 8;
    const int r16 = (r + 15) / 16 * 16;
    const int GP = sp_round_pitch(r16, 8);                   // G pitch == 8 (mod 32): transposed A fragments conflict-free
    float* gs = smem;                                        // [K8][GP]
    float* bs = smem + K8 * GP;                              // [K8][SP_YP]
    const int ky = blockIdx.x; const int64_t b = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    for (int i = tid; i < K8 * GP / 4; i += 128) cp_async_zfill<16>(gs + 4 * i, tab + T.gc + 4 * i, true);     // padded G, as stored
    cp_async_commit();
    for (int i = tid; i < K8 * 64; i += 128) {
        const int k = i >> 6, n = i & 63;
        float v = 0.0f;
        if (k < M2) {
            const int q = k < J ? k : k - J;
            const int64_t o = ((b * J + q) * m + ky) * SP_C + (n & 31);
            if (k < J) v = n < 32 ? __ldg(Or + o) : __ldg(Oi + o);
            else v = n < 32 ? __ldg(Oi + o) : -__ldg(Or + o);
        }
        bs[k * SP_YP + n] = v;
    }
    cp_async_wait<0>();
    __syncthreads();
    float* pb = P + (b * r) * (int64_t)J * SP_C;
    for (int mt = warp; mt < r16 / 16; mt += 4) {
        float acc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][e] = 0.0f;
        const int x0 = mt * 16;
        for (int k0 = 0; k0 < K8; k0 += 8) {
            uint32_t ahi[4], alo[4];
            const float* pa = gs + (k0 + t) * GP + x0 + g;   // A[x][k] = G[k][x]
            split_tf32(pa[0], ahi[0], alo[0]);
            split_tf32(pa[8], ahi[1], alo[1]);
            split_tf32(pa[4 * GP], ahi[2], alo[2]);
            split_tf32(pa[4 * GP + 8], ahi[3], alo[3]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float* p = bs + (k0 + t) * SP_YP + 8 * j + g;
                uint32_t bhi[2], blo[2];
                split_tf32(p[0], bhi[0], blo[0]);
                split_tf32(p[4 * SP_YP], bhi[1], blo[1]);
                mma_tf32(acc[j], alo, bhi);
                mma_tf32(acc[j], ahi, blo);
                mma_tf32(acc[j], ahi, bhi);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int jrow = (j < 4 ? ky : m + ky), c = (8 * j + 2 * t) & 31;
            const int xa = x0 + g, xb = x0 + g + 8;
            if (xa < r) *reinterpret_cast<float2*>(pb + ((int64_t)xa * J + jrow) * SP_C + c) = make_float2(acc[j][0], acc[j][1]);
            if (xb < r) *reinterpret_cast<float2*>(pb + ((int64_t)xb * J + jrow) * SP_C + c) = make_float2(acc[j][2], acc[j][3]);
        }
    }
}

// ------------------------------------------------------------------------------------------------------------
// S3: per (b,x) row and chunk of 32 y:  out[y][o] = act( F3[y][:] * P[:, o] + X[y][:] * Wr[:, o] + br[o] ).
// M = y, N = o (32), K = JP + 32.  One warp per row at a time; X chunks (and the row's P block) are streamed
// through a private double buffer.
// ------------------------------------------------------------------------------------------------------------
template <int KJ>    // k-steps of the spectral part: JP = 8*KJ
__global__ void __launch_bounds__(SP_WARPS * 32, 2)
spectral_inv_y_kernel(const float* __restrict__ X, const float* __restrict__ P, const float* __restrict__ Wr,
                      const float* __restrict__ br, const float* __restrict__ tab, float* __restrict__ out, int r, int m,
                      int act, int64_t nrows) {
    extern __shared__ __align__(16) float smem[];
    const SpecTables T = spec_tables(r, m);
    constexpr int JP = 8 * KJ;
    float* f3 = smem;                                    // [RY][F3P]
    float* wr = f3 + T.RY * T.F3P;                       // [32][40]
    constexpr int XST = SP_YB * SP_XP3;                  // X chunk stage
    constexpr int PST = JP * SP_PP;                      // P row block
    float* wbuf = wr + SP_C * SP_PP + (threadIdx.x >> 5) * (2 * XST + 2 * PST);
    for (int i = threadIdx.x; i < T.RY * T.F3P; i += blockDim.x) f3[i] = __ldg(tab + T.f3 + i);
    for (int i = threadIdx.x; i < SP_C * SP_C; i += blockDim.x) wr[(i / SP_C) * SP_PP + (i % SP_C)] = __ldg(Wr + i);
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // rows of the P blocks beyond J stay zero for the whole kernel (cp.async only ever writes rows < J)
    for (int i = lane; i < 2 * PST; i += 32) wbuf[2 * XST + i] = 0.0f;
    __syncthreads();

    const int nchunk = T.RY / SP_YB;
    const int64_t gw = (int64_t)blockIdx.x * SP_WARPS + (threadIdx.x >> 5);
    const int64_t nw = (int64_t)gridDim.x * SP_WARPS;
    const int64_t my_rows = gw < nrows ? (nrows - gw + nw - 1) / nw : 0;
    const int64_t nitem = my_rows * nchunk;

    auto load = [&](int64_t item, int stage) {
        const int64_t ri = item / nchunk;
        const int64_t row = gw + ri * nw;
        const int chunk = (int)(item % nchunk);
        const int y0 = chunk * SP_YB;
        const float* src = X + row * (int64_t)r * SP_C;
        float* dst = wbuf + stage * XST;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int yy = i * 4 + (lane >> 3), c4 = (lane & 7) * 4;
            const bool ok = y0 + yy < r;
            cp_async_zfill<16>(dst + yy * SP_XP3 + c4, src + (int64_t)(ok ? y0 + yy : 0) * SP_C + c4, ok);
        }
        if (chunk == 0) {                                  // the row's P block [J][32] -> pitch 40
            const float* ps = P + row * (int64_t)T.J * SP_C;
            float* pd = wbuf + 2 * XST + (int)(ri & 1) * PST;
            for (int i = lane; i < T.J * 8; i += 32) {
                const int j = i >> 3, c4 = (i & 7) * 4;
                cp_async_zfill<16>(pd + j * SP_PP + c4, ps + j * SP_C + c4, true);
            }
        }
        cp_async_commit();
    };

    float bias[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) { bias[j][0] = __ldg(br + 8 * j + 2 * t); bias[j][1] = __ldg(br + 8 * j + 2 * t + 1); }

    if (nitem > 0) load(0, 0);
    for (int64_t it = 0; it < nitem; ++it) {
        if (it + 1 < nitem) { load(it + 1, (int)((it + 1) & 1)); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncwarp();
        const int64_t ri = it / nchunk;
        const int chunk = (int)(it % nchunk);
        const float* xs = wbuf + (it & 1) * XST;
        const float* ps = wbuf + 2 * XST + (int)(ri & 1) * PST;
        const float* fs = f3 + chunk * SP_YB * T.F3P;
        float acc[2][4][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.0f;
        // spectral part: A = F3 chunk [32 y][JP], B = P block [JP][32]
#pragma unroll
        for (int k8 = 0; k8 < KJ; ++k8) {
            const int kk = k8 * 8 + t;
            uint32_t ahi[2][4], alo[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float* p = fs + (16 * i + g) * T.F3P + kk;
                split_tf32(p[0], ahi[i][0], alo[i][0]);
                split_tf32(p[8 * T.F3P], ahi[i][1], alo[i][1]);
                split_tf32(p[4], ahi[i][2], alo[i][2]);
                split_tf32(p[8 * T.F3P + 4], ahi[i][3], alo[i][3]);
            }
            uint32_t bhi[4][2], blo[4][2];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* p = ps + kk * SP_PP + 8 * j + g;
                split_tf32(p[0], bhi[j][0], blo[j][0]);
                split_tf32(p[4 * SP_PP], bhi[j][1], blo[j][1]);
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
        // residual part: A = X chunk [32 y][32 i], B = Wr [32 i][32 o]
#pragma unroll
        for (int k8 = 0; k8 < SP_C / 8; ++k8) {
            const int kk = k8 * 8 + t;
            uint32_t ahi[2][4], alo[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float* p = xs + (16 * i + g) * SP_XP3 + kk;
                split_tf32(p[0], ahi[i][0], alo[i][0]);
                split_tf32(p[8 * SP_XP3], ahi[i][1], alo[i][1]);
                split_tf32(p[4], ahi[i][2], alo[i][2]);
                split_tf32(p[8 * SP_XP3 + 4], ahi[i][3], alo[i][3]);
            }
            uint32_t bhi[4][2], blo[4][2];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float* p = wr + kk * SP_PP + 8 * j + g;
                split_tf32(p[0], bhi[j][0], blo[j][0]);
                split_tf32(p[4 * SP_PP], bhi[j][1], blo[j][1]);
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
        const int64_t row = gw + ri * nw;
        float* dst = out + row * (int64_t)r * SP_C;
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int y = chunk * SP_YB + 16 * i + g + 8 * hf;
                if (y < r) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float2 v;
                        v.x = apply_act(acc[i][j][2 * hf] + bias[j][0], act);
                        v.y = apply_act(acc[i][j][2 * hf + 1] + bias[j][1], act);
                        *reinterpret_cast<float2*>(dst + (int64_t)y * SP_C + 8 * j + 2 * t) = v;
                    }
                }
            }
    }
}

template <int NT>
static int launch_fwd_y(const float* x, const float* tab, float* y1, int r, int m, int64_t nrows, cudaStream_t st) {
    static SmemOptIn configured;
    const SpecTables T = spec_tables(r, m);
    const size_t smem = ((size_t)T.RY * T.F1P + (size_t)SP_WARPS * 2 * SP_YB * SP_XP1) * sizeof(float);
    if (smem > 200 * 1024) return SPGT_ERR_SHAPE;
    if (int e = smem_opt_in(spectral_fwd_y_kernel<NT>, smem, configured)) return e;
    const int64_t want = ceil_div(nrows, (int64_t)SP_WARPS);
    const int64_t cap = (int64_t)num_sms() * (smem <= 74 * 1024 ? 3 : 2);
    spectral_fwd_y_kernel<NT><<<(unsigned)(want < cap ? want : cap), SP_WARPS * 32, smem, st>>>(x, tab, y1, r, m, nrows);
    return launch_status();
}

template <int KJ>
static int launch_inv_y(const float* x, const float* p, const float* wr, const float* br, const float* tab, float* out,
                        int r, int m, int act, int64_t nrows, cudaStream_t st) {
    static SmemOptIn configured;
    const SpecTables T = spec_tables(r, m);
    const size_t smem = ((size_t)T.RY * T.F3P + SP_C * SP_PP +
                         (size_t)SP_WARPS * (2 * SP_YB * SP_XP3 + 2 * 8 * KJ * SP_PP)) * sizeof(float);
    if (smem > 200 * 1024) return SPGT_ERR_SHAPE;
    if (int e = smem_opt_in(spectral_inv_y_kernel<KJ>, smem, configured)) return e;
    const int64_t want = ceil_div(nrows, (int64_t)SP_WARPS);
    const int64_t cap = (int64_t)num_sms() * 2;
    spectral_inv_y_kernel<KJ><<<(unsigned)(want < cap ? want : cap), SP_WARPS * 32, smem, st>>>(x, p, wr, br, tab, out, r,
                                                                                              m, act, nrows);
    return launch_status();
}

}  // namespace spgt

using namespace spgt;

static bool spectral_shape_ok(int r, int m) { return r >= 2 && m >= 1 && m <= 16 && 2 * m <= r && r <= 4096; }

extern "C" size_t spgt_spectral_tables_bytes(int r, int m) {
    if (!spectral_shape_ok(r, m)) return 0;
    return (size_t)spec_tables(r, m).total * sizeof(float);
}

extern "C" int spgt_spectral_tables_init(void* tables, size_t tables_bytes, int r, int m, spgt_stream_t stream) {
    if (!tables) return SPGT_ERR_NULL;
    if (!spectral_shape_ok(r, m)) return SPGT_ERR_SHAPE;
    if (tables_bytes < spgt_spectral_tables_bytes(r, m)) return SPGT_ERR_WORKSPACE;
    if (!aligned16(tables)) return SPGT_ERR_ALIGN;
    spectral_tables_kernel<<<64, 256, 0, (cudaStream_t)stream>>>((float*)tables, r, m);
    return launch_status();
}

// workspace layout (floats): Y1 [B,r,J,C] | P [B,r,J,C] | Zr, Zi, Or, Oi [B,J,m,C] each
extern "C" size_t spgt_spectral_workspace_bytes(int B, int r, int m, int C) {
    if (B <= 0 || C != SP_C || !spectral_shape_ok(r, m)) return 0;
    const size_t J = 2 * (size_t)m;
    return ((size_t)2 * B * r * J * C + (size_t)4 * B * J * m * C) * sizeof(float);
}

extern "C" int spgt_spectral_conv2d_fwd(const float* x, const float* wr, const float* br, const float* fw0,
                                        const float* fw1, const void* tables, void* workspace, size_t workspace_bytes,
                                        float* y, int B, int r, int C, int m, int act, spgt_stream_t stream) {
    if (!x || !wr || !br || !fw0 || !fw1 || !tables || !y) return SPGT_ERR_NULL;
    if (B <= 0 || C != SP_C || !spectral_shape_ok(r, m) || act < 0 || act > 3 || B > 65535) return SPGT_ERR_SHAPE;
    const size_t need = spgt_spectral_workspace_bytes(B, r, m, C);
    if (!workspace || workspace_bytes < need) return SPGT_ERR_WORKSPACE;
    if (!aligned16(x) || !aligned16(y) || !aligned16(tables) || !aligned16(workspace) || !aligned16(fw0) || !aligned16(fw1))
        return SPGT_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const SpecTables T = spec_tables(r, m);
    const float* tab = (const float*)tables;
    const size_t J = 2 * (size_t)m;
    float* Y1 = (float*)workspace;
    float* P = Y1 + (size_t)B * r * J * C;
    float* Zr = P + (size_t)B * r * J * C;
    float* Zi = Zr + (size_t)B * J * m * C;
    float* Or = Zi + (size_t)B * J * m * C;
    float* Oi = Or + (size_t)B * J * m * C;
    const int64_t nrows = (int64_t)B * r;
    int e;
    switch (T.JP / 8) {
        case 1: e = launch_fwd_y<1>(x, tab, Y1, r, m, nrows, st); break;
        case 2: e = launch_fwd_y<2>(x, tab, Y1, r, m, nrows, st); break;
        case 3: e = launch_fwd_y<3>(x, tab, Y1, r, m, nrows, st); break;
        default: e = launch_fwd_y<4>(x, tab, Y1, r, m, nrows, st); break;
    }
    if (e) return e;
    const size_t gsmem = (size_t)2 * J * r * sizeof(float);
    if (gsmem > 200 * 1024) return SPGT_ERR_SHAPE;
    static SmemOptIn cfg_a, cfg_c, cfg_am, cfg_cm;
    const bool staged = r <= SP_XMAX;                       // tensor-core S2a / S2c with everything staged in shared memory
    if (staged) {
        const int MT = ceil_div(2 * (int)J, 16), r8 = ceil_div(r, 8) * 8;
        const size_t smem_a = ((size_t)16 * MT * sp_round_pitch(r8, 4) + (size_t)(r8 > 16 * MT ? r8 : 16 * MT) * SP_YP) * sizeof(float);
        if ((e = smem_opt_in(spectral_fwd_x_mma_kernel, smem_a, cfg_am))) return e;
        spectral_fwd_x_mma_kernel<<<dim3(m, B), 128, smem_a, st>>>(Y1, tab, Zr, Zi, r, m);
    } else {
        if ((e = smem_opt_in(spectral_fwd_x_kernel, gsmem, cfg_a))) return e;
        spectral_fwd_x_kernel<<<dim3(m, B), 256, gsmem, st>>>(Y1, tab, Zr, Zi, r, m);
    }
    if ((e = launch_status())) return e;
    spectral_mix_kernel<<<(unsigned)(J * m), 256, 0, st>>>(Zr, Zi, fw0, fw1, Or, Oi, B, m);
    if ((e = launch_status())) return e;
    if (staged) {
        const int K8 = ceil_div(2 * (int)J, 8) * 8, r16 = ceil_div(r, 16) * 16;
        const size_t smem_c = ((size_t)K8 * sp_round_pitch(r16, 8) + (size_t)K8 * SP_YP) * sizeof(float);
        if ((e = smem_opt_in(spectral_inv_x_mma_kernel, smem_c, cfg_cm))) return e;
        spectral_inv_x_mma_kernel<<<dim3(m, B), 128, smem_c, st>>>(Or, Oi, tab, P, r, m);
    } else {
        if ((e = smem_opt_in(spectral_inv_x_kernel, gsmem, cfg_c))) return e;
        spectral_inv_x_kernel<<<dim3(m, B), 256, gsmem, st>>>(Or, Oi, tab, P, r, m);
    }
    if ((e = launch_status())) return e;
    switch (T.JP / 8) {
        case 1: return launch_inv_y<1>(x, P, wr, br, tab, y, r, m, act, nrows, st);
        case 2: return launch_inv_y<2>(x, P, wr, br, tab, y, r, m, act, nrows, st);
        case 3: return launch_inv_y<3>(x, P, wr, br, tab, y, r, m, act, nrows, st);
        default: return launch_inv_y<4>(x, P, wr, br, tab, y, r, m, act, nrows, st);
    }
}
