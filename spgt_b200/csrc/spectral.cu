// FNO2d spectral layer as a mode-truncated DFT.
//
// The reference computes rfft2 over the full r x (r/2+1) spectrum, keeps two m x m corner blocks, mixes channels
// per mode, scatters into a zero spectrum and runs irfft2.  Only 2m x m modes are ever non-zero, so the same
// result is obtained from four small contractions (r may be prime, no FFT factorisation is needed):
//   S1  Y1[b,x,j,c]  = sum_y F1[j,y] X[b,x,y,c]          forward DFT along y, j = (re|im) x ky     [tcgen05 GEMM]
//   S2a Z[b,q,ky,c]  = sum_x G[q,x] Y1c[b,x,ky,c]        forward DFT along x, q = the 2m kept kx   [warp MMA]
//   S2b O[b,q,ky,o]  = sum_i Z[b,q,ky,i] W[q,ky,i,o]     complex channel mixing per mode           [FFMA]
//   S2c P[b,x,j,o]   = sum_q conj(G)[q,x] O[b,q,ky,o]    inverse DFT along x                        [warp MMA]
//   S3  out[b,x,y,o] = act( sum_j F3[y,j] P[b,x,j,o] + sum_i X[b,x,y,i] Wr[i,o] + br[o] )           [tcgen05 GEMM]
// F3 carries the Hermitian-symmetry weights of the real inverse transform (1 for ky = 0, 2 otherwise; the
// imaginary part of the ky = 0 column is ignored exactly as a c2r transform does) and both 1/r normalisations
// of norm='ortho' are folded into F1 and F3.  S1 reads X once, S3 reads X once and writes the output once.
//
// S1 and S3 run on the persistent tcgen05 GEMM kernel of tc_gemm.cu (3xTF32, operands split on the fly): S1 as the GEMM
// D[(x, c)][j] over k = y with the prepared image of F1^T as W, S3 as one GEMM per image row over k = (channel | mode) whose
// W stages are the image of Wr and the image of the row's P block, which S2c writes directly in that layout.
// For r <= 256 the F3 rows stay in tensor memory as a constant A operand and S3's W-loader warp lays out the row's plain P
// block itself; larger r streams F3 through the A rings and reads P as a prepared image.
#include "tc_common.cuh"

namespace spgt {

// tc_gemm.cu
int spectral_tc_prepare(const float* w_kn, int ldw, int K, int N, float* img, cudaStream_t st);
int spectral_fwd_y_tc(const float* x, const float* f1_img, float* y1, int r, int J, int64_t nimg, cudaStream_t st);
int spectral_inv_y_tc(const float* x, const float* f3, const float* wr_img, const float* p_img, const float* p_plain, int J,
                      const float* br, float* out, int r, int64_t nimg, int act, cudaStream_t st);

constexpr int SP_C = 32;         // channel width handled by the tensor-core kernels
constexpr int SP_IMG = 2 * SP_C * TC_BK;   // floats of one W stage image: hi and lo, 32 rows (n) x 32 k each
constexpr int SP_XMAX = 256;      // largest r the staged S2a / S2c kernels accept (shared-memory budget)
__host__ __device__ inline int sp_round_pitch(int n, int rem) {   // smallest p >= n with p % 32 == rem
    int p = (n + 31) / 32 * 32 + rem;
    if (p - 32 >= n) p -= 32;
    return p;
}

struct SpecTables {              // offsets in floats into the table buffer
    int r, m, J, F1P, F3ROWS, KP;
    int f1t, f3, gr, gi, total;
    int GA_ROWS, GA_P, ga, GC_ROWS, GC_P, gc;    // zero-padded copies of G in the shared-memory layouts of S2a / S2c (r <= SP_XMAX)
    int f1img, filled;                           // W image of F1^T (written by the weight-preparation kernel); `filled` = floats the table kernel writes
};
__host__ __device__ inline SpecTables spec_tables(int r, int m) {
    SpecTables t;
    t.r = r; t.m = m; t.J = 2 * m;
    t.F1P = 32;                                   // F1T [r][32]: row y, column j = part * m + ky (re block, then im block)
    t.F3ROWS = (r + 255) / 256 * 256;             // F3 [F3ROWS][32]: row y, column j; zero beyond r and beyond 2m
    t.KP = (r + TC_BK - 1) / TC_BK * TC_BK;
    t.f1t = 0;
    t.f3 = t.f1t + r * t.F1P;
    t.gr = t.f3 + t.F3ROWS * 32;
    t.gi = t.gr + t.J * r;
    t.total = (t.gi + t.J * r + 3) / 4 * 4;
    t.GA_ROWS = (2 * t.J + 15) / 16 * 16; t.GA_P = sp_round_pitch((r + 7) / 8 * 8, 4);
    t.GC_ROWS = (2 * t.J + 7) / 8 * 8;    t.GC_P = sp_round_pitch((r + 15) / 16 * 16, 8);
    t.ga = t.total; t.gc = t.ga;
    if (r <= SP_XMAX) {
        t.gc = t.ga + t.GA_ROWS * t.GA_P;
        t.total = t.gc + t.GC_ROWS * t.GC_P;
    }
    t.filled = t.total = (t.total + 3) / 4 * 4;
    t.f1img = t.total;
    t.total += 2 * 32 * t.KP;
    return t;
}

__device__ __forceinline__ int kept_kx(int q, int r, int m) { return q < m ? q : r - 2 * m + q; }

__global__ void spectral_tables_kernel(float* tab, int r, int m) {
    const SpecTables T = spec_tables(r, m);
    const int n = T.filled;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        float v = 0.0f;
        if (i < T.f3) {                                        // F1T[y][j]
            const int y = i / T.F1P, j = i % T.F1P;
            if (j < T.J) {
                const int ky = j < m ? j : j - m;
                double s, c;
                sincospi(2.0 * (double)(((int64_t)ky * y) % r) / (double)r, &s, &c);
                v = (float)((j < m ? c : -s) / (double)r);
            }
        } else if (i < T.gr) {                                 // F3[y][j]
            const int k = i - T.f3;
            const int y = k / 32, j = k % 32;
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
                    const float* __restrict__ fw1, float* __restrict__ Or, float* __restrict__ Oi, int B, int m,
                    const float* __restrict__ wr, float* __restrict__ wr_img) {
    __shared__ float2 w[SP_C * SP_C];
    if (blockIdx.x == 0 && wr_img != nullptr)            // W stage image of the residual weight Wr [i][o] for the y-inverse GEMM
        for (int i = threadIdx.x; i < SP_C * SP_C; i += blockDim.x) tc_img_store(wr_img, SP_C, i % SP_C, i / SP_C, __ldg(wr + i));
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

// S2c for large r: P[b,x,ky,o] + i P[b,x,m+ky,o] = sum_q conj(G[q,x]) * O[b,q,ky,o], written into the W stage image of
// image row (b, x), element (n = o, k = j).   grid (m, B), lane = o, warp = x stride 8.
__global__ void __launch_bounds__(256)
spectral_inv_x_kernel(const float* __restrict__ Or, const float* __restrict__ Oi, const float* __restrict__ tab,
                      float* __restrict__ Pimg, int r, int m) {
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
        float* img = Pimg + (b * r + x) * (int64_t)SP_IMG;
        tc_img_store(img, SP_C, lane, ky, pr);
        tc_img_store(img, SP_C, lane, m + ky, pi);
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
// owns a slice of the output (S2a: 8 columns, S2c: every eighth 16-row tile); eight warps per CTA.
// ------------------------------------------------------------------------------------------------------------
constexpr int SP_YP = 72;         // pitch of the [x][64] / [k][64] B operands, == 8 (mod 32)


__global__ void __launch_bounds__(256)
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
    for (int i = tid; i < r8 * 16; i += 256) {
        const int x = i >> 4, c4 = i & 15;
        const bool ok = x < r;
        const float* src = yb + ((int64_t)(ok ? x : 0) * J + (c4 < 8 ? ky : m + ky)) * SP_C + (c4 & 7) * 4;
        cp_async_zfill<16>(ys + x * SP_YP + c4 * 4, src, ok);
    }
    cp_async_commit();
    for (int i = tid; i < 16 * MT * GP / 4; i += 256) cp_async_zfill<16>(gs + 4 * i, tab + T.ga + 4 * i, true);   // padded G, as stored
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    float acc[4][1][4];             // eight warps, eight columns each
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 1; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;
    const int n0 = warp * 8;
    for (int k0 = 0; k0 < r8; k0 += 8) {
        uint32_t bhi[1][2], blo[1][2];
#pragma unroll
        for (int j = 0; j < 1; ++j) {
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
                for (int j = 0; j < 1; ++j) {
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
            for (int j = 0; j < 1; ++j) {
                const int row = 16 * i + g, col = n0 + 8 * j + 2 * t;
                *reinterpret_cast<float2*>(rs + row * SP_YP + col) = make_float2(acc[i][j][0], acc[i][j][1]);
                *reinterpret_cast<float2*>(rs + (row + 8) * SP_YP + col) = make_float2(acc[i][j][2], acc[i][j][3]);
            }
        }
    __syncthreads();
    for (int e = tid; e < J * SP_C; e += 256) {
        const int q = e >> 5, c = e & 31;
        const int64_t o = ((b * J + q) * m + ky) * SP_C + c;
        Zr[o] = rs[q * SP_YP + c] - rs[(J + q) * SP_YP + 32 + c];
        Zi[o] = rs[q * SP_YP + 32 + c] + rs[(J + q) * SP_YP + c];
    }
}

__global__ void __launch_bounds__(256)
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
    for (int i = tid; i < K8 * GP / 4; i += 256) cp_async_zfill<16>(gs + 4 * i, tab + T.gc + 4 * i, true);     // padded G, as stored
    cp_async_commit();
    for (int i = tid; i < K8 * 64; i += 256) {
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
    for (int mt = warp; mt < r16 / 16; mt += 8) {
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


// The layer can be run in chunks of samples, each through all its kernels before the next, so that S3's second read of a
// chunk's X (r * r * 32 floats per sample) finds it in L2.  On B200 the fixed cost of the extra launches of the two
// persistent GEMM kernels outweighs the saved DRAM reads at the sizes measured (chunks of 8 samples at r = 211: 0.89 ms
// against 0.45 ms for 64 samples), so the default chunk is the whole batch; "spectral_chunk_mb" sets a limit in MB of X.
static int g_spectral_chunk_mb = 0;          // 0 = no chunking
void spectral_set_chunk_mb(int mb) { g_spectral_chunk_mb = mb; }
static int spectral_chunk(int r) {
    if (g_spectral_chunk_mb <= 0) return 65535;
    const int64_t per_sample = (int64_t)r * r * SP_C * 4;
    int64_t n = ((int64_t)g_spectral_chunk_mb << 20) / per_sample;
    return (int)(n < 1 ? 1 : (n > 65535 ? 65535 : n));
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
    const SpecTables T = spec_tables(r, m);
    spectral_tables_kernel<<<64, 256, 0, (cudaStream_t)stream>>>((float*)tables, r, m);
    if (int e = launch_status()) return e;
    return spectral_tc_prepare((const float*)tables + T.f1t, T.F1P, r, T.J, (float*)tables + T.f1img, (cudaStream_t)stream);
}

extern "C" int spgt_spectral_chunk_samples(int r) { return r >= 2 ? spectral_chunk(r) : 0; }

// kernels one call of spgt_spectral_conv2d_fwd launches: five per chunk of samples
extern "C" int spgt_spectral_launches(int B, int r, int m) {
    if (B <= 0 || !spectral_shape_ok(r, m)) return 0;
    return 5 * ceil_div(B, spectral_chunk(r));
}

// floats of the P blocks of one image row: plain [J][32] for r <= 256, a W stage image for larger r
static size_t spectral_p_floats(int r, int J) { return r <= 256 ? (size_t)J * SP_C : (size_t)SP_IMG; }

// workspace layout (floats), sized for one chunk of CH samples: Y1 [CH,r,J,C] | P [CH,r][p_floats] | Zr, Zi, Or, Oi [CH,J,m,C] each | Wr image
extern "C" size_t spgt_spectral_workspace_bytes(int B, int r, int m, int C) {
    if (B <= 0 || C != SP_C || !spectral_shape_ok(r, m)) return 0;
    const size_t J = 2 * (size_t)m, CH = (size_t)(B < spectral_chunk(r) ? B : spectral_chunk(r));
    return (CH * r * J * C + CH * r * spectral_p_floats(r, (int)J) + (size_t)4 * CH * J * m * C + SP_IMG) * sizeof(float);
}

extern "C" int spgt_spectral_conv2d_fwd(const float* x, const float* wr, const float* br, const float* fw0,
                                        const float* fw1, const void* tables, void* workspace, size_t workspace_bytes,
                                        float* y, int B, int r, int C, int m, int act, spgt_stream_t stream) {
    if (!x || !wr || !br || !fw0 || !fw1 || !tables || !y) return SPGT_ERR_NULL;
    if (B <= 0 || C != SP_C || !spectral_shape_ok(r, m) || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    const size_t need = spgt_spectral_workspace_bytes(B, r, m, C);
    if (!workspace || workspace_bytes < need) return SPGT_ERR_WORKSPACE;
    if (!aligned16(x) || !aligned16(y) || !aligned16(tables) || !aligned16(workspace) || !aligned16(fw0) || !aligned16(fw1))
        return SPGT_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const SpecTables T = spec_tables(r, m);
    const float* tab = (const float*)tables;
    const size_t J = 2 * (size_t)m;
    const int CH = B < spectral_chunk(r) ? B : spectral_chunk(r);
    if (CH > 65535) return SPGT_ERR_SHAPE;                  // (grid y dimension of the x-transform kernels)
    float* Y1 = (float*)workspace;
    float* P = Y1 + (size_t)CH * r * J * C;
    float* Zr = P + (size_t)CH * r * spectral_p_floats(r, (int)J);
    float* Zi = Zr + (size_t)CH * J * m * C;
    float* Or = Zi + (size_t)CH * J * m * C;
    float* Oi = Or + (size_t)CH * J * m * C;
    float* wr_img = Oi + (size_t)CH * J * m * C;
    const size_t gsmem = (size_t)2 * J * r * sizeof(float);
    if (gsmem > 200 * 1024) return SPGT_ERR_SHAPE;
    static SmemOptIn cfg_a, cfg_c, cfg_am, cfg_cm;
    const bool staged = r <= SP_XMAX;                       // tensor-core S2a / S2c with everything staged in shared memory
    // Large r: S2c writes W stage images, columns k < 2m only; the k padding must be zero (it meets zero columns of F3, but
    // 0 * NaN would still spoil the sum), so the images are cleared first.
    if (!staged && cudaMemsetAsync(P, 0, (size_t)CH * r * SP_IMG * sizeof(float), st) != cudaSuccess) return launch_status();
    int e;
    for (int b0 = 0; b0 < B; b0 += CH) {
        const int nb = B - b0 < CH ? B - b0 : CH;
        const float* xc = x + (size_t)b0 * r * r * C;
        float* yc = y + (size_t)b0 * r * r * C;
        const int64_t nimg = (int64_t)nb * r;
        if ((e = spectral_fwd_y_tc(xc, tab + T.f1img, Y1, r, (int)J, nimg, st))) return e;
        if (staged) {
            const int MT = ceil_div(2 * (int)J, 16), r8 = ceil_div(r, 8) * 8;
            const size_t smem_a = ((size_t)16 * MT * sp_round_pitch(r8, 4) + (size_t)(r8 > 16 * MT ? r8 : 16 * MT) * SP_YP) * sizeof(float);
            if ((e = smem_opt_in(spectral_fwd_x_mma_kernel, smem_a, cfg_am))) return e;
            spectral_fwd_x_mma_kernel<<<dim3(m, nb), 256, smem_a, st>>>(Y1, tab, Zr, Zi, r, m);
        } else {
            if ((e = smem_opt_in(spectral_fwd_x_kernel, gsmem, cfg_a))) return e;
            spectral_fwd_x_kernel<<<dim3(m, nb), 256, gsmem, st>>>(Y1, tab, Zr, Zi, r, m);
        }
        if ((e = launch_status())) return e;
        spectral_mix_kernel<<<(unsigned)(J * m), 256, 0, st>>>(Zr, Zi, fw0, fw1, Or, Oi, nb, m, wr, b0 == 0 ? wr_img : nullptr);
        if ((e = launch_status())) return e;
        if (staged) {
            const int K8 = ceil_div(2 * (int)J, 8) * 8, r16 = ceil_div(r, 16) * 16;
            const size_t smem_c = ((size_t)K8 * sp_round_pitch(r16, 8) + (size_t)K8 * SP_YP) * sizeof(float);
            if ((e = smem_opt_in(spectral_inv_x_mma_kernel, smem_c, cfg_cm))) return e;
            spectral_inv_x_mma_kernel<<<dim3(m, nb), 256, smem_c, st>>>(Or, Oi, tab, P, r, m);
        } else {
            if ((e = smem_opt_in(spectral_inv_x_kernel, gsmem, cfg_c))) return e;
            spectral_inv_x_kernel<<<dim3(m, nb), 256, gsmem, st>>>(Or, Oi, tab, P, r, m);
        }
        if ((e = launch_status())) return e;
        if ((e = spectral_inv_y_tc(xc, tab + T.f3, wr_img, P, P, (int)J, br, yc, r, nimg, act, st))) return e;
    }
    return SPGT_OK;
}
