// Interpolation kernels of the down- and up-scaler (bilinear, align_corners=True, NHWC), fused with the
// neighbouring element-wise work.  All are bandwidth-bound gather + lerp kernels with 16-byte accesses.
#include "common.cuh"

namespace spgt {

// Source coordinate exactly as ATen computes it in fp32: scale = (in-1)/(out-1), src = scale*dst,
// i0 = min(int(src), in-1), lambda = clamp(src - i0, 0, 1), i1 = i0 + (i0 < in-1).
struct Tap { int i0, i1; float w0, w1; };
__host__ __device__ __forceinline__ Tap make_tap(int dst, int in_size, int out_size) {
    Tap tp;
    if (in_size == out_size) { tp.i0 = tp.i1 = dst; tp.w0 = 1.0f; tp.w1 = 0.0f; return tp; }
    const float scale = out_size > 1 ? (float)(in_size - 1) / (float)(out_size - 1) : 0.0f;
    const float src = scale * (float)dst;
    int i0 = (int)src;
    if (i0 > in_size - 1) i0 = in_size - 1;
    float lam = src - (float)i0;
    lam = fminf(fmaxf(lam, 0.0f), 1.0f);
    tp.i0 = i0; tp.i1 = i0 + (i0 < in_size - 1 ? 1 : 0); tp.w1 = lam; tp.w0 = 1.0f - lam;
    return tp;
}

// The three gather + lerp kernels below give one output row (b, yo) to a block at a time: the row tap is computed once,
// the position inside the row needs only 32-bit arithmetic, and consecutive threads write consecutive float4s.
__global__ void __launch_bounds__(256)
bilinear_kernel(const float4* __restrict__ x, float4* __restrict__ y, int Hi, int Wi, int Ho, int Wo, int C4, int act,
                int rows) {
    const int per_row = Wo * C4;
    const bool fixed_c = (blockDim.x % C4) == 0;          // a thread keeps its channel quad: no division per element
    const int c_fix = threadIdx.x % C4, x_step = blockDim.x / C4;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int b = row / Ho, yo = row - b * Ho;
        const Tap ty = make_tap(yo, Hi, Ho);
        const float4* r0 = x + ((int64_t)b * Hi + ty.i0) * Wi * C4;
        const float4* r1 = x + ((int64_t)b * Hi + ty.i1) * Wi * C4;
        float4* yr = y + (int64_t)row * per_row;
        int xo = threadIdx.x / C4;
        for (int e = threadIdx.x; e < per_row; e += blockDim.x, xo += x_step) {
            int c = c_fix;
            if (!fixed_c) { xo = e / C4; c = e - xo * C4; }
            const Tap tx = make_tap(xo, Wi, Wo);
            const float4 v00 = __ldg(r0 + tx.i0 * C4 + c);
            const float4 v01 = __ldg(r0 + tx.i1 * C4 + c);
            const float4 v10 = __ldg(r1 + tx.i0 * C4 + c);
            const float4 v11 = __ldg(r1 + tx.i1 * C4 + c);
            const float w00 = ty.w0 * tx.w0, w01 = ty.w0 * tx.w1, w10 = ty.w1 * tx.w0, w11 = ty.w1 * tx.w1;
            float4 o;
            o.x = apply_act(v00.x * w00 + v01.x * w01 + v10.x * w10 + v11.x * w11, act);
            o.y = apply_act(v00.y * w00 + v01.y * w01 + v10.y * w10 + v11.y * w11, act);
            o.z = apply_act(v00.z * w00 + v01.z * w01 + v10.z * w10 + v11.z * w11, act);
            o.w = apply_act(v00.w * w00 + v01.w * w01 + v10.w * w10 + v11.w * w11, act);
            yr[e] = o;
        }
    }
}

// y[b,yo,xo,c] = act( lerp over the 4 taps of act(conv3x3(node)[tap] + bias[c]) ).
// A block handles C0_PIX consecutive output pixels: the 4x4 input patch around each pixel's taps (zero padded
// outside the image) and the four lerp weights are staged once in shared memory, then thread c evaluates the
// convolution of channel c at the taps whose weight is non-zero (for exact 2:1 down-scaling that is one tap).
// The activation is a template parameter (the kernel is bound by its instruction count: a run-time switch per element
// costs a fifth of it), and the per-pixel index arithmetic (two divisions, two taps) is done once per pixel, not once
// per patch element.
constexpr int C0_PIX = 32;
template <int ACT>
__global__ void __launch_bounds__(128)
conv0_down_kernel(const float* __restrict__ node, const float4* __restrict__ w, const float4* __restrict__ bias,
                  float4* __restrict__ y, int Hi, int Wi, int Ho, int Wo, int CQ, int npix) {
    constexpr int act = ACT;
    __shared__ __align__(16) float patch[C0_PIX][16];
    __shared__ __align__(16) float wt[C0_PIX][4];
    __shared__ int pix_row0[C0_PIX], pix_y0[C0_PIX], pix_x0[C0_PIX];    // b * Hi, first tap row - 1, first tap column - 1
    const bool fixed_cq = (128 % CQ) == 0;            // every item of a thread has the same channel quad: keep its weights in registers
    float4 wk[9], bc;
    if (fixed_cq) {
        const int cq = threadIdx.x % CQ;
#pragma unroll
        for (int k = 0; k < 9; ++k) wk[k] = __ldg(w + k * CQ + cq);
        bc = __ldg(bias + cq);
    }
    for (int p0 = blockIdx.x * C0_PIX; p0 < npix; p0 += gridDim.x * C0_PIX) {
        __syncthreads();                              // the previous group's patch has been consumed
        if (threadIdx.x < C0_PIX) {
            const int pi = threadIdx.x, p = p0 + pi;
            if (p < npix) {
                const int t2 = p / Wo, xo = p - t2 * Wo;
                const int b = t2 / Ho, yo = t2 - b * Ho;
                const Tap ty = make_tap(yo, Hi, Ho), tx = make_tap(xo, Wi, Wo);
                pix_row0[pi] = b * Hi; pix_y0[pi] = ty.i0 - 1; pix_x0[pi] = tx.i0 - 1;
                // a clamped second tap (i1 == i0) reads the same pixel: fold its weight into the first tap
                const float wy0 = ty.i1 == ty.i0 ? ty.w0 + ty.w1 : ty.w0, wy1 = ty.i1 == ty.i0 ? 0.0f : ty.w1;
                const float wx0 = tx.i1 == tx.i0 ? tx.w0 + tx.w1 : tx.w0, wx1 = tx.i1 == tx.i0 ? 0.0f : tx.w1;
                *reinterpret_cast<float4*>(&wt[pi][0]) = make_float4(wy0 * wx0, wy0 * wx1, wy1 * wx0, wy1 * wx1);
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < C0_PIX * 16; i += blockDim.x) {
            const int pi = i >> 4, e = i & 15;
            float v = 0.0f;
            if (p0 + pi < npix) {
                const int yy = pix_y0[pi] + (e >> 2), xx = pix_x0[pi] + (e & 3);
                if (yy >= 0 && yy < Hi && xx >= 0 && xx < Wi) v = __ldg(node + ((int64_t)pix_row0[pi] + yy) * Wi + xx);
            }
            patch[pi][e] = v;
        }
        __syncthreads();
        for (int item = threadIdx.x; item < C0_PIX * CQ; item += blockDim.x) {
            const int pi = item / CQ, cq = item - pi * CQ;
            const int p = p0 + pi;
            if (p >= npix) break;
            if (!fixed_cq) {
#pragma unroll
                for (int k = 0; k < 9; ++k) wk[k] = __ldg(w + k * CQ + cq);
                bc = __ldg(bias + cq);
            }
            float pv[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 r = *reinterpret_cast<const float4*>(&patch[pi][4 * q]);
                pv[4 * q] = r.x; pv[4 * q + 1] = r.y; pv[4 * q + 2] = r.z; pv[4 * q + 3] = r.w;
            }
            const float4 wv = *reinterpret_cast<const float4*>(&wt[pi][0]);
            const float wgt4[4] = {wv.x, wv.y, wv.z, wv.w};
            float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int d = 0; d < 2; ++d) {
                    const float wgt = wgt4[a * 2 + d];
                    if (wgt != 0.0f) {
                        float4 s4 = bc;
#pragma unroll
                        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                            for (int kx = 0; kx < 3; ++kx) {
                                const float pvv = pv[(a + ky) * 4 + d + kx];
                                const float4 ww = wk[ky * 3 + kx];
                                s4.x = fmaf(pvv, ww.x, s4.x); s4.y = fmaf(pvv, ww.y, s4.y);
                                s4.z = fmaf(pvv, ww.z, s4.z); s4.w = fmaf(pvv, ww.w, s4.w);
                            }
                        o.x = fmaf(apply_act(s4.x, act), wgt, o.x); o.y = fmaf(apply_act(s4.y, act), wgt, o.y);
                        o.z = fmaf(apply_act(s4.z, act), wgt, o.z); o.w = fmaf(apply_act(s4.w, act), wgt, o.w);
                    }
                }
            o.x = apply_act(o.x, act); o.y = apply_act(o.y, act); o.z = apply_act(o.z, act); o.w = apply_act(o.w, act);
            y[(int64_t)p * CQ + cq] = o;
        }
    }
}

// y[b,yo,xo,:] = bilinear(uw)[b,yo,xo,:] + grid[b,yo,xo,0]*wg[0,:] + grid[b,yo,xo,1]*wg[1,:] + bias
__global__ void __launch_bounds__(256)
upsample_grid_kernel(const float4* __restrict__ uw, const float2* __restrict__ grid, const float4* __restrict__ wg,
                     const float4* __restrict__ bias, float4* __restrict__ y, int Hi, int Wi, int Ho, int Wo, int C4,
                     int rows) {
    const int per_row = Wo * C4;
    // When the block size is a multiple of C4 a thread keeps its channel quad for every element: the three parameter
    // vectors stay in registers and the pixel index advances by a constant, without a division.
    const bool fixed_c = (blockDim.x % C4) == 0;
    const int c_fix = threadIdx.x % C4, x_fix = threadIdx.x / C4, x_step = blockDim.x / C4;
    float4 g0f, g1f, bbf;
    if (fixed_c) { g0f = __ldg(wg + c_fix); g1f = __ldg(wg + C4 + c_fix); bbf = __ldg(bias + c_fix); }
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int b = row / Ho, yo = row - b * Ho;
        const Tap ty = make_tap(yo, Hi, Ho);
        const float4* r0 = uw + ((int64_t)b * Hi + ty.i0) * Wi * C4;
        const float4* r1 = uw + ((int64_t)b * Hi + ty.i1) * Wi * C4;
        const float2* gr = grid + (int64_t)row * Wo;
        float4* yr = y + (int64_t)row * per_row;
        int xo = x_fix;
        for (int e = threadIdx.x; e < per_row; e += blockDim.x, xo += x_step) {
            int c = c_fix;
            float4 g0 = g0f, g1 = g1f, bb = bbf;
            if (!fixed_c) {
                xo = e / C4; c = e - xo * C4;
                g0 = __ldg(wg + c); g1 = __ldg(wg + C4 + c); bb = __ldg(bias + c);
            }
            const Tap tx = make_tap(xo, Wi, Wo);
            const float4 v00 = __ldg(r0 + tx.i0 * C4 + c);
            const float4 v01 = __ldg(r0 + tx.i1 * C4 + c);
            const float4 v10 = __ldg(r1 + tx.i0 * C4 + c);
            const float4 v11 = __ldg(r1 + tx.i1 * C4 + c);
            const float w00 = ty.w0 * tx.w0, w01 = ty.w0 * tx.w1, w10 = ty.w1 * tx.w0, w11 = ty.w1 * tx.w1;
            const float2 gxy = __ldg(gr + xo);
            float4 o;
            o.x = v00.x * w00 + v01.x * w01 + v10.x * w10 + v11.x * w11 + gxy.x * g0.x + gxy.y * g1.x + bb.x;
            o.y = v00.y * w00 + v01.y * w01 + v10.y * w10 + v11.y * w11 + gxy.x * g0.y + gxy.y * g1.y + bb.y;
            o.z = v00.z * w00 + v01.z * w01 + v10.z * w10 + v11.z * w11 + gxy.x * g0.z + gxy.y * g1.z + bb.z;
            o.w = v00.w * w00 + v01.w * w01 + v10.w * w10 + v11.w * w11 + gxy.x * g0.w + gxy.y * g1.w + bb.w;
            yr[e] = o;
        }
    }
}

// Up-sampling variant of the two kernels above (MODE 0: bilinear_kernel, MODE 1: upsample_grid_kernel, the same
// arithmetic in the same order).  When the output has more rows than the input every source row is a tap of several
// output rows and every source pixel of several output pixels; gathered straight from global memory most of those
// reads miss L1 and the kernel runs at the L2 rate.  Here a block takes G consecutive output rows of one image,
// copies the few source rows they need (contiguous in NHWC) into shared memory once with 16-byte cp.async, and lerps
// from there: global reads are ns / G source rows per output row, all coalesced.
constexpr int LS_THREADS = 512;
template <int MODE>
__global__ void __launch_bounds__(LS_THREADS)
lerp_staged_kernel(const float4* __restrict__ x, float4* __restrict__ y, int Hi, int Wi, int Ho, int Wo, int C4, int act,
                   const float2* __restrict__ grid, const float4* __restrict__ wg, const float4* __restrict__ bias, int G,
                   int groups_per_img, int n_groups) {
    extern __shared__ float4 srow[];                       // the source rows of the current group
    const int row_f4 = Wi * C4, per_row = Wo * C4;
    const int c = threadIdx.x % C4, x0 = threadIdx.x / C4, x_step = blockDim.x / C4;     // blockDim.x % C4 == 0 (host)
    float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0, bb = g0;
    if (MODE == 1) { g0 = __ldg(wg + c); g1 = __ldg(wg + C4 + c); bb = __ldg(bias + c); }
    for (int grp = blockIdx.x; grp < n_groups; grp += gridDim.x) {
        const int b = grp / groups_per_img, y0 = (grp - b * groups_per_img) * G;
        const int y1 = y0 + G < Ho ? y0 + G : Ho;
        const int s_lo = make_tap(y0, Hi, Ho).i0, s_hi = make_tap(y1 - 1, Hi, Ho).i1;
        const float4* src = x + ((int64_t)b * Hi + s_lo) * row_f4;
        __syncthreads();                                   // the previous group has been read
        for (int i = threadIdx.x; i < (s_hi - s_lo + 1) * row_f4; i += blockDim.x) cp_async_zfill<16>(srow + i, src + i, true);
        cp_async_commit();
        cp_async_wait_all();
        __syncthreads();
        for (int yo = y0; yo < y1; ++yo) {
            const Tap ty = make_tap(yo, Hi, Ho);
            const float4* r0 = srow + (ty.i0 - s_lo) * row_f4;
            const float4* r1 = srow + (ty.i1 - s_lo) * row_f4;
            const int64_t row = (int64_t)b * Ho + yo;
            float4* yr = y + row * per_row;
            const float2* gr = MODE == 1 ? grid + row * Wo : nullptr;
            int xo = x0;
            for (int e = threadIdx.x; e < per_row; e += blockDim.x, xo += x_step) {
                const Tap tx = make_tap(xo, Wi, Wo);
                const float4 v00 = r0[tx.i0 * C4 + c], v01 = r0[tx.i1 * C4 + c];
                const float4 v10 = r1[tx.i0 * C4 + c], v11 = r1[tx.i1 * C4 + c];
                const float w00 = ty.w0 * tx.w0, w01 = ty.w0 * tx.w1, w10 = ty.w1 * tx.w0, w11 = ty.w1 * tx.w1;
                float4 o;
                if (MODE == 1) {
                    const float2 gxy = __ldg(gr + xo);
                    o.x = v00.x * w00 + v01.x * w01 + v10.x * w10 + v11.x * w11 + gxy.x * g0.x + gxy.y * g1.x + bb.x;
                    o.y = v00.y * w00 + v01.y * w01 + v10.y * w10 + v11.y * w11 + gxy.x * g0.y + gxy.y * g1.y + bb.y;
                    o.z = v00.z * w00 + v01.z * w01 + v10.z * w10 + v11.z * w11 + gxy.x * g0.z + gxy.y * g1.z + bb.z;
                    o.w = v00.w * w00 + v01.w * w01 + v10.w * w10 + v11.w * w11 + gxy.x * g0.w + gxy.y * g1.w + bb.w;
                } else {
                    o.x = apply_act(v00.x * w00 + v01.x * w01 + v10.x * w10 + v11.x * w11, act);
                    o.y = apply_act(v00.y * w00 + v01.y * w01 + v10.y * w10 + v11.y * w11, act);
                    o.z = apply_act(v00.z * w00 + v01.z * w01 + v10.z * w10 + v11.z * w11, act);
                    o.w = apply_act(v00.w * w00 + v01.w * w01 + v10.w * w10 + v11.w * w11, act);
                }
                yr[e] = o;
            }
        }
    }
}

static unsigned grid_for(int64_t items, int threads, int per_sm) {
    const int64_t want = ceil_div(items, (int64_t)threads);
    const int64_t cap = (int64_t)num_sms() * per_sm;
    return (unsigned)(want < cap ? want : cap);
}

// Rows per group and shared-memory bytes of lerp_staged_kernel for an up-sampling shape, or G = 0 when the gather
// kernels should be used (down-sampling, channel counts that do not divide the block, rows too long).
struct StagedPlan { int G; size_t smem; };
static StagedPlan staged_plan(int Hi, int Wi, int Ho, int C4) {
    StagedPlan p{0, 0};
    if (Ho <= Hi || (LS_THREADS / 2) % C4 != 0) return p;
    const size_t row_bytes = (size_t)Wi * C4 * sizeof(float4);
    for (int G = 4; G >= 2; G -= 2) {
        int ns = 0;
        for (int y0 = 0; y0 < Ho; y0 += G) {
            const int y1 = y0 + G < Ho ? y0 + G : Ho;
            const int n = make_tap(y1 - 1, Hi, Ho).i1 - make_tap(y0, Hi, Ho).i0 + 1;
            if (n > ns) ns = n;
        }
        if (ns * row_bytes <= (G == 4 ? 48u : 100u) * 1024u) { p.G = G; p.smem = ns * row_bytes; return p; }
    }
    return p;
}
template <int MODE>
static int launch_staged(const StagedPlan& p, const float4* x, float4* y, int B, int Hi, int Wi, int Ho, int Wo, int C4, int act,
                         const float2* grid, const float4* wg, const float4* bias, cudaStream_t st) {
    static SmemOptIn configured;
    if (int e = smem_opt_in(lerp_staged_kernel<MODE>, p.smem, configured)) return e;
    const int gpi = ceil_div(Ho, p.G);
    const int64_t n_groups = (int64_t)B * gpi;
    const int per_sm = (int)(200 * 1024 / (p.smem + 1024));
    // few resident blocks (long rows): larger blocks keep enough threads per SM (measured: 512 better above 48 KB, worse below)
    const int threads = (p.smem > 48 * 1024 && LS_THREADS % (2 * C4) == 0) ? LS_THREADS : LS_THREADS / 2;
    lerp_staged_kernel<MODE><<<grid_for(n_groups, 1, per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm)), threads, p.smem, st>>>(
        x, y, Hi, Wi, Ho, Wo, C4, act, grid, wg, bias, p.G, gpi, (int)n_groups);
    return launch_status();
}

// y[b,yo,xo,:] = act(bilinear(concat(x1[..., :c1], x2[..., :c2], x3[..., :c3])))  -- the three sources keep their own
// (padded) channel pitch, the output is dense.  One thread per (pixel, 4 output channels), scalar gathers.
__global__ void __launch_bounds__(256)
bilinear_concat3_kernel(const float* __restrict__ x1, const float* __restrict__ x2, const float* __restrict__ x3, int p1,
                        int p2, int p3, int c1, int c2, int c3, float4* __restrict__ y, int Hi, int Wi, int Ho, int Wo,
                        int act, int rows) {
    const int C4 = (c1 + c2 + c3) / 4;
    const int per_row = Wo * C4;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int b = row / Ho, yo = row - b * Ho;
        const Tap ty = make_tap(yo, Hi, Ho);
        const int64_t q0 = ((int64_t)b * Hi + ty.i0) * Wi, q1 = ((int64_t)b * Hi + ty.i1) * Wi;
        float4* yr = y + (int64_t)row * per_row;
        for (int e = threadIdx.x; e < per_row; e += blockDim.x) {
            const int xo = e / C4, cg = e - xo * C4;
            const Tap tx = make_tap(xo, Wi, Wo);
            const float w00 = ty.w0 * tx.w0, w01 = ty.w0 * tx.w1, w10 = ty.w1 * tx.w0, w11 = ty.w1 * tx.w1;
            const int64_t o00 = q0 + tx.i0, o01 = q0 + tx.i1, o10 = q1 + tx.i0, o11 = q1 + tx.i1;
            float o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                int c = cg * 4 + k;
                const float* src; int pitch;
                if (c < c1) { src = x1; pitch = p1; }
                else if (c < c1 + c2) { src = x2; pitch = p2; c -= c1; }
                else { src = x3; pitch = p3; c -= c1 + c2; }
                const float v = __ldg(src + o00 * pitch + c) * w00 + __ldg(src + o01 * pitch + c) * w01 +
                                __ldg(src + o10 * pitch + c) * w10 + __ldg(src + o11 * pitch + c) * w11;
                o[k] = apply_act(v, act);
            }
            yr[e] = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

}  // namespace spgt

using namespace spgt;

extern "C" int spgt_bilinear_fwd(const float* x, float* y, int B, int Hi, int Wi, int Ho, int Wo, int C, int act,
                                 spgt_stream_t stream) {
    if (!x || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hi <= 0 || Wi <= 0 || Ho <= 0 || Wo <= 0 || C <= 0 || (C & 3) || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(y)) return SPGT_ERR_ALIGN;
    const int64_t rows = (int64_t)B * Ho;
    if (rows > 0x7fffffffLL || (int64_t)Wo * (C / 4) > 0x7fffffffLL || (int64_t)Wi * (C / 4) > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    const StagedPlan plan = staged_plan(Hi, Wi, Ho, C / 4);
    if (plan.G > 0)
        return launch_staged<0>(plan, reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), B, Hi, Wi, Ho, Wo, C / 4, act,
                                nullptr, nullptr, nullptr, (cudaStream_t)stream);
    bilinear_kernel<<<grid_for(rows, 1, 8), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), Hi, Wi, Ho, Wo, C / 4, act, (int)rows);
    return launch_status();
}

extern "C" int spgt_bilinear_concat3_fwd(const float* x1, const float* x2, const float* x3, int p1, int p2, int p3, int c1,
                                         int c2, int c3, float* y, int B, int Hi, int Wi, int Ho, int Wo, int act,
                                         spgt_stream_t stream) {
    if (!x1 || !x2 || !x3 || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hi <= 0 || Wi <= 0 || Ho <= 0 || Wo <= 0 || c1 <= 0 || c2 <= 0 || c3 <= 0 || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if (p1 < c1 || p2 < c2 || p3 < c3 || ((c1 + c2 + c3) & 3)) return SPGT_ERR_SHAPE;
    if (!aligned16(y)) return SPGT_ERR_ALIGN;
    const int64_t rows = (int64_t)B * Ho;
    if (rows > 0x7fffffffLL || (int64_t)Wo * (c1 + c2 + c3) > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    bilinear_concat3_kernel<<<grid_for(rows, 1, 8), 256, 0, (cudaStream_t)stream>>>(
        x1, x2, x3, p1, p2, p3, c1, c2, c3, reinterpret_cast<float4*>(y), Hi, Wi, Ho, Wo, act, (int)rows);
    return launch_status();
}

extern "C" int spgt_conv0_down_fwd(const float* node, const float* w, const float* bias, float* y, int B, int Hi, int Wi,
                                   int Ho, int Wo, int Cout, int act, spgt_stream_t stream) {
    if (!node || !w || !bias || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hi <= 0 || Wi <= 0 || Ho <= 0 || Wo <= 0 || Cout <= 0 || (Cout & 3) || Cout > 512 || act < 0 || act > 3)
        return SPGT_ERR_SHAPE;
    const int64_t npix = (int64_t)B * Ho * Wo;
    if (npix > 0x7fffffffLL - 64 * 1024 * 1024) return SPGT_ERR_SHAPE;
    if (!aligned16(w) || !aligned16(bias) || !aligned16(y)) return SPGT_ERR_ALIGN;
    const unsigned grid = grid_for(ceil_div(npix, (int64_t)C0_PIX), 1, 16);
    auto launch = [&](auto kern) {
        kern<<<grid, 128, 0, (cudaStream_t)stream>>>(node, reinterpret_cast<const float4*>(w), reinterpret_cast<const float4*>(bias),
                                                     reinterpret_cast<float4*>(y), Hi, Wi, Ho, Wo, Cout / 4, (int)npix);
    };
    switch (act) {
        case SPGT_ACT_RELU: launch(conv0_down_kernel<SPGT_ACT_RELU>); break;
        case SPGT_ACT_SILU: launch(conv0_down_kernel<SPGT_ACT_SILU>); break;
        case SPGT_ACT_SILU2: launch(conv0_down_kernel<SPGT_ACT_SILU2>); break;
        default: launch(conv0_down_kernel<SPGT_ACT_NONE>); break;
    }
    return launch_status();
}

extern "C" int spgt_upsample_grid_fwd(const float* uw, const float* grid, const float* wg, const float* bias, float* y,
                                      int B, int Hi, int Wi, int Ho, int Wo, int C, spgt_stream_t stream) {
    if (!uw || !grid || !wg || !bias || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hi <= 0 || Wi <= 0 || Ho <= 0 || Wo <= 0 || C <= 0 || (C & 3)) return SPGT_ERR_SHAPE;
    if (!aligned16(uw) || !aligned16(grid) || !aligned16(wg) || !aligned16(bias) || !aligned16(y)) return SPGT_ERR_ALIGN;
    const int64_t rows = (int64_t)B * Ho;
    if (rows > 0x7fffffffLL || (int64_t)Wo * (C / 4) > 0x7fffffffLL || (int64_t)Wi * (C / 4) > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    const StagedPlan plan = staged_plan(Hi, Wi, Ho, C / 4);
    if (plan.G > 0)
        return launch_staged<1>(plan, reinterpret_cast<const float4*>(uw), reinterpret_cast<float4*>(y), B, Hi, Wi, Ho, Wo, C / 4, 0,
                                reinterpret_cast<const float2*>(grid), reinterpret_cast<const float4*>(wg),
                                reinterpret_cast<const float4*>(bias), (cudaStream_t)stream);
    upsample_grid_kernel<<<grid_for(rows, 1, 8), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4*>(uw), reinterpret_cast<const float2*>(grid), reinterpret_cast<const float4*>(wg),
        reinterpret_cast<const float4*>(bias), reinterpret_cast<float4*>(y), Hi, Wi, Ho, Wo, C / 4, (int)rows);
    return launch_status();
}
