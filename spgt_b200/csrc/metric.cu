// Relative L2 error per sample:  e[n] = sqrt( mean((pred - target)^2) / (mean(target^2) + eps) ).
// This is the validation metric of the reference (engine/metric.py:47-67 with alpha = 0, beta = 1: the per-sample
// `loss` before the 'L1' / 'L2' / 'Linf' reduction over samples).  One block per sample, fixed reduction order:
// the result is bitwise reproducible.
#include "common.cuh"

namespace spgt {

__global__ void __launch_bounds__(1024)
relative_l2_kernel(const float* __restrict__ pred, const float* __restrict__ target, float* __restrict__ out,
                   int64_t n_per_sample, float eps) {
    __shared__ float sd[32], st[32];
    const float* p = pred + blockIdx.x * n_per_sample;
    const float* t = target + blockIdx.x * n_per_sample;
    float d2 = 0.0f, t2 = 0.0f;
    for (int64_t i = threadIdx.x; i < n_per_sample; i += blockDim.x) {
        const float tv = __ldg(t + i), dv = __ldg(p + i) - tv;
        d2 = fmaf(dv, dv, d2);
        t2 = fmaf(tv, tv, t2);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        d2 += __shfl_xor_sync(0xffffffffu, d2, o);
        t2 += __shfl_xor_sync(0xffffffffu, t2, o);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sd[warp] = d2; st[warp] = t2; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        d2 = lane < nw ? sd[lane] : 0.0f;
        t2 = lane < nw ? st[lane] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            d2 += __shfl_xor_sync(0xffffffffu, d2, o);
            t2 += __shfl_xor_sync(0xffffffffu, t2, o);
        }
        if (lane == 0) {
            const float inv = 1.0f / (float)n_per_sample;
            out[blockIdx.x] = sqrtf((d2 * inv) / (t2 * inv + eps));
        }
    }
}

}  // namespace spgt

using namespace spgt;

extern "C" int spgt_relative_l2_fwd(const float* pred, const float* target, float* per_sample, int N, int64_t n_per_sample,
                                    float eps, spgt_stream_t stream) {
    if (!pred || !target || !per_sample) return SPGT_ERR_NULL;
    if (N <= 0 || n_per_sample <= 0) return SPGT_ERR_SHAPE;
    relative_l2_kernel<<<(unsigned)N, 1024, 0, (cudaStream_t)stream>>>(pred, target, per_sample, n_per_sample, eps);
    return launch_status();
}
