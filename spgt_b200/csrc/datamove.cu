// Data-movement kernels: batched 2-D transpose (fp32) and the dual corner-block gather / scatter of the
// spectral layer (complex64).  All are pure copies, so results are bit-exact.
#include "common.cuh"

namespace spgt {

// dst[b][n][m] = src[b][m][n].  32x32 tiles through padded shared memory: 128-byte coalesced rows on both
// the load and the store side.  Tiles are flattened into blockIdx.x so that no grid dimension overflows.
__global__ void __launch_bounds__(256) batched_transpose_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                                 int M, int N, int tiles_m, int tiles_n) {
    __shared__ float tile[32][33];
    const int64_t t = blockIdx.x;
    const int tn = (int)(t % tiles_n);
    const int tm = (int)((t / tiles_n) % tiles_m);
    const int64_t b = t / ((int64_t)tiles_n * tiles_m);
    const float* s = src + b * (int64_t)M * N;
    float* d = dst + b * (int64_t)M * N;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = tm * 32 + ty + 8 * i, n = tn * 32 + tx;
        if (m < M && n < N) tile[ty + 8 * i][tx] = __ldg(s + (int64_t)m * N + n);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int n = tn * 32 + ty + 8 * i, m = tm * 32 + tx;
        if (m < M && n < N) d[(int64_t)n * M + m] = tile[tx][ty + 8 * i];
    }
}

// out_k[(h*W_low + w)*dim + c] = src[c*H_all*W_all + (hb_k + h)*W_all + wb_k + w], k = blockIdx.z.
// Tile = 32 positions (h,w) x 32 channels c of float2.
__global__ void __launch_bounds__(256) gather_dual_kernel(const float2* __restrict__ src, float2* __restrict__ out1,
                                                           float2* __restrict__ out2, int dim, int H_all, int W_all,
                                                           int H_low, int W_low, int hb1, int wb1, int hb2, int wb2) {
    __shared__ float2 tile[32][33];
    const int which = blockIdx.z;
    const int hb = which ? hb2 : hb1, wb = which ? wb2 : wb1;
    float2* out = which ? out2 : out1;
    const int P = H_low * W_low;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < 4; ++i) {   // load: consecutive threads walk positions (contiguous along w in src)
        const int c = c0 + ty + 8 * i, p = p0 + tx;
        if (c < dim && p < P) {
            const int h = p / W_low, w = p - h * W_low;
            tile[ty + 8 * i][tx] = __ldg(src + (int64_t)c * H_all * W_all + (int64_t)(hb + h) * W_all + wb + w);
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {   // store: consecutive threads walk channels (contiguous in out)
        const int p = p0 + ty + 8 * i, c = c0 + tx;
        if (c < dim && p < P) out[(int64_t)p * dim + c] = tile[tx][ty + 8 * i];
    }
}

// One thread per element of out [dim, H_all, W_all]: the value from block 2, else block 1, else zero.
__global__ void __launch_bounds__(256) scatter_dual_kernel(const float2* __restrict__ src1, const float2* __restrict__ src2,
                                                            float2* __restrict__ out, int dim, int H_all, int W_all,
                                                            int H_low, int W_low, int hb1, int wb1, int hb2, int wb2,
                                                            int64_t total) {
    const int64_t plane = (int64_t)H_all * W_all;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int c = (int)(i / plane);
        const int rem = (int)(i - (int64_t)c * plane);
        const int h = rem / W_all, w = rem - h * W_all;
        float2 v = make_float2(0.0f, 0.0f);
        const int h2 = h - hb2, w2 = w - wb2, h1 = h - hb1, w1 = w - wb1;
        if (h2 >= 0 && h2 < H_low && w2 >= 0 && w2 < W_low) {
            v = __ldg(src2 + ((int64_t)h2 * W_low + w2) * dim + c);
        } else if (h1 >= 0 && h1 < H_low && w1 >= 0 && w1 < W_low) {
            v = __ldg(src1 + ((int64_t)h1 * W_low + w1) * dim + c);
        }
        out[i] = v;
    }
}

}  // namespace spgt

using namespace spgt;

extern "C" int spgt_batched_transpose(const float* src, float* dst, int M, int N, int batch, spgt_stream_t stream) {
    if (!src || !dst) return SPGT_ERR_NULL;
    if (M <= 0 || N <= 0 || batch <= 0) return SPGT_ERR_SHAPE;
    const int tiles_m = ceil_div(M, 32), tiles_n = ceil_div(N, 32);
    const int64_t blocks = (int64_t)tiles_m * tiles_n * batch;
    if (blocks > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    batched_transpose_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(src, dst, M, N, tiles_m, tiles_n);
    return launch_status();
}

static int check_blocks(int dim, int H_all, int W_all, int H_low, int W_low, int hb1, int wb1, int hb2, int wb2) {
    if (dim <= 0 || H_all <= 0 || W_all <= 0 || H_low <= 0 || W_low <= 0) return SPGT_ERR_SHAPE;
    if (hb1 < 0 || wb1 < 0 || hb2 < 0 || wb2 < 0) return SPGT_ERR_SHAPE;
    if (hb1 + H_low > H_all || hb2 + H_low > H_all || wb1 + W_low > W_all || wb2 + W_low > W_all) return SPGT_ERR_SHAPE;
    return SPGT_OK;
}

extern "C" int spgt_transpose_gather_dual(const float* src, float* out1, float* out2, int dim, int H_all, int W_all,
                                          int H_low, int W_low, int hb1, int wb1, int hb2, int wb2,
                                          spgt_stream_t stream) {
    if (!src || !out1 || !out2) return SPGT_ERR_NULL;
    if (int e = check_blocks(dim, H_all, W_all, H_low, W_low, hb1, wb1, hb2, wb2)) return e;
    dim3 grid(ceil_div(H_low * W_low, 32), ceil_div(dim, 32), 2);
    if (grid.y > 65535u) return SPGT_ERR_SHAPE;
    gather_dual_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float2*>(src), reinterpret_cast<float2*>(out1), reinterpret_cast<float2*>(out2), dim,
        H_all, W_all, H_low, W_low, hb1, wb1, hb2, wb2);
    return launch_status();
}

extern "C" int spgt_transpose_scatter_dual(const float* src1, const float* src2, float* out, int dim, int H_all,
                                           int W_all, int H_low, int W_low, int hb1, int wb1, int hb2, int wb2,
                                           spgt_stream_t stream) {
    if (!src1 || !src2 || !out) return SPGT_ERR_NULL;
    if (int e = check_blocks(dim, H_all, W_all, H_low, W_low, hb1, wb1, hb2, wb2)) return e;
    const int64_t total = (int64_t)dim * H_all * W_all;
    const int64_t want = ceil_div(total, (int64_t)256);
    const unsigned blocks = (unsigned)(want < (int64_t)num_sms() * 16 ? want : (int64_t)num_sms() * 16);
    scatter_dual_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float2*>(src1), reinterpret_cast<const float2*>(src2), reinterpret_cast<float2*>(out),
        dim, H_all, W_all, H_low, W_low, hb1, wb1, hb2, wb2, total);
    return launch_status();
}
