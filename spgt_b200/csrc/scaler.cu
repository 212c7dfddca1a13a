// Interpolation kernels of the down- and up-scaler (bilinear, align_corners=True, NHWC), fused with the
// neighbouring element-wise work.  All are bandwidth-bound gather + lerp kernels with 16-byte accesses.
#include "common.cuh"

namespace spgt {

// Source coordinate exactly as ATen computes it in fp32: scale = (in-1)/(out-1), src = scale*dst,
// i0 = min(int(src), in-1), lambda = clamp(src - i0, 0, 1), i1 = i0 + (i0 < in-1).
struct Tap { int i0, i1; float w0, w1; };
__device__ __forceinline__ Tap make_tap(int dst, int in_size, int out_size) {
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

__global__ void __launch_bounds__(256)
bilinear_kernel(const float4* __restrict__ x, float4* __restrict__ y, int Hi, int Wi, int Ho, int Wo, int C4, int act,
                int64_t total) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C4);
        int64_t p = i / C4;
        const int xo = (int)(p % Wo); p /= Wo;
        const int yo = (int)(p % Ho);
        const int64_t b = p / Ho;
        const Tap ty = make_tap(yo, Hi, Ho), tx = make_tap(xo, Wi, Wo);
        const float4* base = x + b * (int64_t)Hi * Wi * C4 + c;
        const float4 v00 = __ldg(base + ((int64_t)ty.i0 * Wi + tx.i0) * C4);
        const float4 v01 = __ldg(base + ((int64_t)ty.i0 * Wi + tx.i1) * C4);
        const float4 v10 = __ldg(base + ((int64_t)ty.i1 * Wi + tx.i0) * C4);
        const float4 v11 = __ldg(base + ((int64_t)ty.i1 * Wi + tx.i1) * C4);
        const float w00 = ty.w0 * tx.w0, w01 = ty.w0 * tx.w1, w10 = ty.w1 * tx.w0, w11 = ty.w1 * tx.w1;
        float4 o;
        o.x = apply_act(v00.x * w00 + v01.x * w01 + v10.x * w10 + v11.x * w11, act);
        o.y = apply_act(v00.y * w00 + v01.y * w01 + v10.y * w10 + v11.y * w11, act);
        o.z = apply_act(v00.z * w00 + v01.z * w01 + v10.z * w10 + v11.z * w11, act);
        o.w = apply_act(v00.w * w00 + v01.w * w01 + v10.w * w10 + v11.w * w11, act);
        y[i] = o;
    }
}

// y[b,yo,xo,c] = act( lerp over the 4 taps of act(conv3x3(node)[tap] + bias[c]) ).
// A block handles C0_PIX consecutive output pixels: the 4x4 input patch around each pixel's taps (zero padded
// outside the image) and the four lerp weights are staged once in shared memory, then thread c evaluates the
// convolution of channel c at the taps whose weight is non-zero (for exact 2:1 down-scaling that is one tap).
constexpr int C0_PIX = 16;
__global__ void __launch_bounds__(128)
conv0_down_kernel(const float* __restrict__ node, const float* __restrict__ w, const float* __restrict__ bias,
                  float* __restrict__ y, int Hi, int Wi, int Ho, int Wo, int Cout, int act, int64_t npix) {
    __shared__ float patch[C0_PIX][16];
    __shared__ float wt[C0_PIX][4];
    const int64_t p0 = (int64_t)blockIdx.x * C0_PIX;
    for (int i = threadIdx.x; i < C0_PIX * 16; i += blockDim.x) {
        const int pi = i >> 4, e = i & 15;
        const int64_t p = p0 + pi;
        float v = 0.0f;
        if (p < npix) {
            const int xo = (int)(p % Wo);
            const int yo = (int)((p / Wo) % Ho);
            const int64_t b = p / ((int64_t)Wo * Ho);
            const Tap ty = make_tap(yo, Hi, Ho), tx = make_tap(xo, Wi, Wo);
            const int yy = ty.i0 - 1 + (e >> 2), xx = tx.i0 - 1 + (e & 3);
            if (yy >= 0 && yy < Hi && xx >= 0 && xx < Wi) v = __ldg(node + (b * Hi + yy) * (int64_t)Wi + xx);
            if (e < 4) {
                // a clamped second tap (i1 == i0) reads the same pixel: fold its weight into the first tap
                const float wy0 = ty.i1 == ty.i0 ? ty.w0 + ty.w1 : ty.w0, wy1 = ty.i1 == ty.i0 ? 0.0f : ty.w1;
                const float wx0 = tx.i1 == tx.i0 ? tx.w0 + tx.w1 : tx.w0, wx1 = tx.i1 == tx.i0 ? 0.0f : tx.w1;
                wt[pi][e] = ((e >> 1) ? wy1 : wy0) * ((e & 1) ? wx1 : wx0);
            }
        }
        patch[pi][e] = v;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < Cout; c += blockDim.x) {
        float wk[9];
#pragma unroll
        for (int k = 0; k < 9; ++k) wk[k] = __ldg(w + k * Cout + c);
        const float bc = __ldg(bias + c);
#pragma unroll 2
        for (int pi = 0; pi < C0_PIX; ++pi) {
            const int64_t p = p0 + pi;
            if (p >= npix) break;
            float pv[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 r = *reinterpret_cast<const float4*>(&patch[pi][4 * q]);
                pv[4 * q] = r.x; pv[4 * q + 1] = r.y; pv[4 * q + 2] = r.z; pv[4 * q + 3] = r.w;
            }
            float o = 0.0f;
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
                for (int d = 0; d < 2; ++d) {
                    const float wgt = wt[pi][a * 2 + d];
                    if (wgt != 0.0f) {
                        float s = bc;
#pragma unroll
                        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                            for (int kx = 0; kx < 3; ++kx) s = fmaf(pv[(a + ky) * 4 + d + kx], wk[ky * 3 + kx], s);
                        o = fmaf(apply_act(s, act), wgt, o);
                    }
                }
            y[p * Cout + c] = apply_act(o, act);
        }
    }
}

// y[b,yo,xo,:] = bilinear(uw)[b,yo,xo,:] + grid[b,yo,xo,0]*wg[0,:] + grid[b,yo,xo,1]*wg[1,:] + bias
__global__ void __launch_bounds__(256)
upsample_grid_kernel(const float4* __restrict__ uw, const float2* __restrict__ grid, const float4* __restrict__ wg,
                     const float4* __restrict__ bias, float4* __restrict__ y, int Hi, int Wi, int Ho, int Wo, int C4,
                     int64_t total) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C4);
        const int64_t pix = i / C4;
        int64_t p = pix;
        const int xo = (int)(p % Wo); p /= Wo;
        const int yo = (int)(p % Ho);
        const int64_t b = p / Ho;
        const Tap ty = make_tap(yo, Hi, Ho), tx = make_tap(xo, Wi, Wo);
        const float4* base = uw + b * (int64_t)Hi * Wi * C4 + c;
        const float4 v00 = __ldg(base + ((int64_t)ty.i0 * Wi + tx.i0) * C4);
        const float4 v01 = __ldg(base + ((int64_t)ty.i0 * Wi + tx.i1) * C4);
        const float4 v10 = __ldg(base + ((int64_t)ty.i1 * Wi + tx.i0) * C4);
        const float4 v11 = __ldg(base + ((int64_t)ty.i1 * Wi + tx.i1) * C4);
        const float w00 = ty.w0 * tx.w0, w01 = ty.w0 * tx.w1, w10 = ty.w1 * tx.w0, w11 = ty.w1 * tx.w1;
        const float2 gxy = __ldg(grid + pix);
        const float4 g0 = __ldg(wg + c), g1 = __ldg(wg + C4 + c), bb = __ldg(bias + c);
        float4 o;
        o.x = v00.x * w00 + v01.x * w01 + v10.x * w10 + v11.x * w11 + gxy.x * g0.x + gxy.y * g1.x + bb.x;
        o.y = v00.y * w00 + v01.y * w01 + v10.y * w10 + v11.y * w11 + gxy.x * g0.y + gxy.y * g1.y + bb.y;
        o.z = v00.z * w00 + v01.z * w01 + v10.z * w10 + v11.z * w11 + gxy.x * g0.z + gxy.y * g1.z + bb.z;
        o.w = v00.w * w00 + v01.w * w01 + v10.w * w10 + v11.w * w11 + gxy.x * g0.w + gxy.y * g1.w + bb.w;
        y[i] = o;
    }
}

// y[b,yo,xo,:] = act(bilinear(concat(x1[..., :c1], x2[..., :c2], x3[..., :c3])))  -- the three sources keep their own
// (padded) channel pitch, the output is dense.  One thread per (pixel, 4 output channels), scalar gathers.
__global__ void __launch_bounds__(256)
bilinear_concat3_kernel(const float* __restrict__ x1, const float* __restrict__ x2, const float* __restrict__ x3, int p1,
                        int p2, int p3, int c1, int c2, int c3, float4* __restrict__ y, int Hi, int Wi, int Ho, int Wo,
                        int act, int64_t total) {
    const int C4 = (c1 + c2 + c3) / 4;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int cg = (int)(i % C4);
        int64_t p = i / C4;
        const int xo = (int)(p % Wo); p /= Wo;
        const int yo = (int)(p % Ho);
        const int64_t b = p / Ho;
        const Tap ty = make_tap(yo, Hi, Ho), tx = make_tap(xo, Wi, Wo);
        const float w00 = ty.w0 * tx.w0, w01 = ty.w0 * tx.w1, w10 = ty.w1 * tx.w0, w11 = ty.w1 * tx.w1;
        const int64_t o00 = (b * Hi + ty.i0) * Wi + tx.i0, o01 = (b * Hi + ty.i0) * Wi + tx.i1;
        const int64_t o10 = (b * Hi + ty.i1) * Wi + tx.i0, o11 = (b * Hi + ty.i1) * Wi + tx.i1;
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
        y[i] = make_float4(o[0], o[1], o[2], o[3]);
    }
}

static unsigned grid_for(int64_t items, int threads, int per_sm) {
    const int64_t want = ceil_div(items, (int64_t)threads);
    const int64_t cap = (int64_t)num_sms() * per_sm;
    return (unsigned)(want < cap ? want : cap);
}

}  // namespace spgt

using namespace spgt;

extern "C" int spgt_bilinear_fwd(const float* x, float* y, int B, int Hi, int Wi, int Ho, int Wo, int C, int act,
                                 spgt_stream_t stream) {
    if (!x || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hi <= 0 || Wi <= 0 || Ho <= 0 || Wo <= 0 || C <= 0 || (C & 3) || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(y)) return SPGT_ERR_ALIGN;
    const int64_t total = (int64_t)B * Ho * Wo * (C / 4);
    bilinear_kernel<<<grid_for(total, 256, 16), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y), Hi, Wi, Ho, Wo, C / 4, act, total);
    return launch_status();
}

extern "C" int spgt_bilinear_concat3_fwd(const float* x1, const float* x2, const float* x3, int p1, int p2, int p3, int c1,
                                         int c2, int c3, float* y, int B, int Hi, int Wi, int Ho, int Wo, int act,
                                         spgt_stream_t stream) {
    if (!x1 || !x2 || !x3 || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hi <= 0 || Wi <= 0 || Ho <= 0 || Wo <= 0 || c1 <= 0 || c2 <= 0 || c3 <= 0 || act < 0 || act > 3) return SPGT_ERR_SHAPE;
    if (p1 < c1 || p2 < c2 || p3 < c3 || ((c1 + c2 + c3) & 3)) return SPGT_ERR_SHAPE;
    if (!aligned16(y)) return SPGT_ERR_ALIGN;
    const int64_t total = (int64_t)B * Ho * Wo * ((c1 + c2 + c3) / 4);
    bilinear_concat3_kernel<<<grid_for(total, 256, 16), 256, 0, (cudaStream_t)stream>>>(
        x1, x2, x3, p1, p2, p3, c1, c2, c3, reinterpret_cast<float4*>(y), Hi, Wi, Ho, Wo, act, total);
    return launch_status();
}

extern "C" int spgt_conv0_down_fwd(const float* node, const float* w, const float* bias, float* y, int B, int Hi, int Wi,
                                   int Ho, int Wo, int Cout, int act, spgt_stream_t stream) {
    if (!node || !w || !bias || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hi <= 0 || Wi <= 0 || Ho <= 0 || Wo <= 0 || Cout <= 0 || (Cout & 3) || Cout > 512 || act < 0 || act > 3)
        return SPGT_ERR_SHAPE;
    const int64_t npix = (int64_t)B * Ho * Wo;
    const int64_t blocks = ceil_div(npix, (int64_t)C0_PIX);
    if (blocks > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    conv0_down_kernel<<<(unsigned)blocks, 128, 0, (cudaStream_t)stream>>>(node, w, bias, y, Hi, Wi, Ho, Wo, Cout, act, npix);
    return launch_status();
}

extern "C" int spgt_upsample_grid_fwd(const float* uw, const float* grid, const float* wg, const float* bias, float* y,
                                      int B, int Hi, int Wi, int Ho, int Wo, int C, spgt_stream_t stream) {
    if (!uw || !grid || !wg || !bias || !y) return SPGT_ERR_NULL;
    if (B <= 0 || Hi <= 0 || Wi <= 0 || Ho <= 0 || Wo <= 0 || C <= 0 || (C & 3)) return SPGT_ERR_SHAPE;
    if (!aligned16(uw) || !aligned16(grid) || !aligned16(wg) || !aligned16(bias) || !aligned16(y)) return SPGT_ERR_ALIGN;
    const int64_t total = (int64_t)B * Ho * Wo * (C / 4);
    upsample_grid_kernel<<<grid_for(total, 256, 16), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4*>(uw), reinterpret_cast<const float2*>(grid), reinterpret_cast<const float4*>(wg),
        reinterpret_cast<const float4*>(bias), reinterpret_cast<float4*>(y), Hi, Wi, Ho, Wo, C / 4, total);
    return launch_status();
}
