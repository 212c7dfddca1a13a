// Backward of the multi-head projection (+ per-head LayerNorm) + position op, element-wise part.
// Reference: multihead_projection_with_position_rrc_backward / multihead_projection_layernorm_with_position_rrc_backward
// (extension/bind/galerkin_attention.cu:26-48, 70-102) and lnorm_grad_ccc_cuda (extension/native/multihead_dim32.cu).
//
// Forward:  h = x W + b  [rows = B*S, D = H*32];  per (row, head): hat = (h - mu) * invsigma, y = hat * lnw + lnb;
//           out[b, h, d_pos + c, s] = y[b*S + s, 32 h + c]  (position rows carry no gradient).
// This kernel takes grad_out [B, H, d_pos + 32, S] and the recomputed h and produces
//   dh [rows, D]  (the gradient with respect to h, row-major: the A operand of the two GEMMs dX = dh W^T and dW = x^T dh),
//   per-block partial sums of  db = sum_rows dh,  dlnw = sum_rows g * hat,  dlnb = sum_rows g   (g = gathered grad_out),
// which a second kernel adds up in block order (deterministic).  Without LayerNorm (lnw == nullptr) dh = g.
// One block = 32 consecutive grid nodes of one sample, all heads; warp w of 4 = head w... for H heads the block has H warps.
#include "common.cuh"

namespace spgt {

constexpr int PB_ROWS = 32;      // grid nodes per block

__global__ void __launch_bounds__(256)
proj_bwd_kernel(const float* __restrict__ grad_out, const float* __restrict__ h, const float* __restrict__ lnw,
                float* __restrict__ dh, float* __restrict__ partial, int S, int H, int d_pos, float eps, int blocks_per_sample) {
    extern __shared__ float tile[];                       // [H*32 channels][33]
    const int b = blockIdx.x / blocks_per_sample;
    const int s0 = (blockIdx.x % blocks_per_sample) * PB_ROWS;
    const int D = H * 32, dpk = d_pos + 32;
    const int lane = threadIdx.x & 31, head = threadIdx.x >> 5;
    // gather: channel c of head hd, node s0 + lane (coalesced along s)
    for (int c = 0; c < 32; ++c) {
        const int s = s0 + lane;
        tile[(head * 32 + c) * 33 + lane] = s < S ? __ldg(grad_out + (((int64_t)b * H + head) * dpk + d_pos + c) * S + s) : 0.0f;
    }
    __syncthreads();
    const int ch = head * 32 + lane;                      // this thread's channel
    const float w = lnw != nullptr ? __ldg(lnw + ch) : 1.0f;
    float acc_db = 0.0f, acc_w = 0.0f, acc_b = 0.0f;
    for (int r = 0; r < PB_ROWS; ++r) {
        const int s = s0 + r;
        if (s >= S) break;
        const int64_t row = (int64_t)b * S + s;
        const float g = tile[ch * 33 + r];
        float d;
        if (lnw != nullptr) {
            const float hv = __ldg(h + row * D + ch);
            float mu = hv;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mu += __shfl_xor_sync(0xffffffffu, mu, o);
            mu *= (1.0f / 32.0f);
            const float cen = hv - mu;
            float var = cen * cen;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
            const float inv = rsqrtf(var * (1.0f / 32.0f) + eps);
            const float hat = cen * inv;
            const float dhat = g * w;
            float m1 = dhat, m2 = dhat * hat;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) { m1 += __shfl_xor_sync(0xffffffffu, m1, o); m2 += __shfl_xor_sync(0xffffffffu, m2, o); }
            d = inv * (dhat - m1 * (1.0f / 32.0f) - hat * m2 * (1.0f / 32.0f));
            acc_w = fmaf(g, hat, acc_w);
            acc_b += g;
        } else {
            d = g;
        }
        dh[row * D + ch] = d;
        acc_db += d;
    }
    float* p = partial + (int64_t)blockIdx.x * 3 * D;
    p[ch] = acc_db; p[D + ch] = acc_w; p[2 * D + ch] = acc_b;
}

__global__ void __launch_bounds__(256)
proj_bwd_reduce_kernel(const float* __restrict__ partial, float* __restrict__ db, float* __restrict__ dlnw, float* __restrict__ dlnb,
                       int D, int nblocks) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 3 * D) return;
    float s = 0.0f;
    for (int k = 0; k < nblocks; ++k) s += __ldg(partial + (int64_t)k * 3 * D + i);
    float* dst = i < D ? db : (i < 2 * D ? dlnw : dlnb);
    if (dst != nullptr) dst[i % D] = s;
}

}  // namespace spgt

using namespace spgt;

extern "C" size_t spgt_projpos_bwd_workspace_bytes(int B, int S, int H) {
    if (B <= 0 || S <= 0 || H <= 0 || H > 8) return 0;
    return (size_t)B * ceil_div(S, PB_ROWS) * 3 * H * 32 * sizeof(float);
}

extern "C" int spgt_projpos_bwd_elementwise(const float* grad_out, const float* h, const float* ln_weight, float eps, float* dh,
                                            float* db, float* dlnw, float* dlnb, int B, int S, int H, int d_head, int d_pos,
                                            void* workspace, size_t workspace_bytes, spgt_stream_t stream) {
    if (!grad_out || !dh) return SPGT_ERR_NULL;
    if (ln_weight && !h) return SPGT_ERR_NULL;
    if (B <= 0 || S <= 0 || H <= 0 || H > 8 || d_head != 32 || d_pos < 0 || d_pos > 8) return SPGT_ERR_SHAPE;
    const int bps = ceil_div(S, PB_ROWS);
    const int64_t nblocks = (int64_t)B * bps;
    if (nblocks > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    if (!workspace || workspace_bytes < spgt_projpos_bwd_workspace_bytes(B, S, H)) return SPGT_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    const int D = H * 32;
    proj_bwd_kernel<<<(unsigned)nblocks, H * 32, (size_t)D * 33 * sizeof(float), st>>>(grad_out, h, ln_weight, dh, (float*)workspace,
                                                                                       S, H, d_pos, eps, bps);
    if (int e = launch_status()) return e;
    proj_bwd_reduce_kernel<<<ceil_div(3 * D, 256), 256, 0, st>>>((const float*)workspace, db, ln_weight ? dlnw : nullptr,
                                                                ln_weight ? dlnb : nullptr, D, (int)nblocks);
    return launch_status();
}
