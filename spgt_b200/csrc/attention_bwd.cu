// Backward of the Galerkin attention op  out[s][j] = sum_i Q[i][s] T[i][j],  T[i][j] = (1/S) sum_s K[i][s] V[j][s]
// (reference: multihead_galerkin_attention_cccr_backward, extension/bind/galerkin_attention.cu:126-173, which runs
// three split-K and three small-K SGEMMs).  Here two kernels, exact fp32 FMA arithmetic:
//   reduce  every CTA streams one chunk of the S columns of a (batch, head) once and accumulates the two dpk x dpk
//           matrices that the gradients need,  T  and  dT[i][j] = sum_s Q[i][s] dOut[s][j],  into its slot of the workspace;
//   apply   every CTA sums the chunk partials in chunk order (deterministic), then, one grid node per thread,
//           dQ[i][s] = sum_j T[i][j] dOut[s][j],   dK[i][s] = (1/S) sum_j dT[i][j] V[j][s],   dV[j][s] = (1/S) sum_i dT[i][j] K[i][s].
// Layouts as in the forward: Q, K, V, dQ, dK, dV [B*H, dpk, S] (S fastest), dOut [B*H, S, dpk].
#include "common.cuh"

namespace spgt {

constexpr int AB_MAXD = 35, AB_TP = 36;        // dpk <= 35; pitch of the dpk x dpk matrices
constexpr int AB_COLS = 64;                    // columns per staged tile of the reduce kernel
constexpr int AB_THREADS = 256;

// workspace per (bh, chunk): T partial [36*36] | dT partial [36*36]
__global__ void __launch_bounds__(AB_THREADS)
attn_bwd_reduce_kernel(const float* __restrict__ Q, const float* __restrict__ K, const float* __restrict__ V,
                       const float* __restrict__ dOut, float* __restrict__ ws, int D, int S, int chunks) {
    __shared__ float ks[AB_MAXD][AB_COLS + 1], vs[AB_MAXD][AB_COLS + 1], qs[AB_MAXD][AB_COLS + 1], gs[AB_COLS][AB_TP + 1];
    const int64_t bh = blockIdx.x / chunks;
    const int chunk = blockIdx.x % chunks;
    const int64_t base = bh * (int64_t)D * S;
    const int ncol_tiles = (S + AB_COLS - 1) / AB_COLS;
    const int t_begin = (int)(((int64_t)chunk * ncol_tiles) / chunks), t_end = (int)(((int64_t)(chunk + 1) * ncol_tiles) / chunks);
    // each thread owns up to 5 entries e = tid + 256 n of the D x D matrices
    float accT[5] = {0, 0, 0, 0, 0}, accD[5] = {0, 0, 0, 0, 0};
    int ei[5], ej[5];
#pragma unroll
    for (int n = 0; n < 5; ++n) { const int e = threadIdx.x + AB_THREADS * n; ei[n] = e < D * D ? e / D : -1; ej[n] = e < D * D ? e % D : 0; }
    for (int tile = t_begin; tile < t_end; ++tile) {
        const int s0 = tile * AB_COLS;
        __syncthreads();
        for (int i = threadIdx.x; i < D * AB_COLS; i += AB_THREADS) {
            const int r = i / AB_COLS, c = i % AB_COLS;
            const bool ok = s0 + c < S;
            const int64_t o = base + (int64_t)r * S + s0 + c;
            ks[r][c] = ok ? __ldg(K + o) : 0.0f;
            vs[r][c] = ok ? __ldg(V + o) : 0.0f;
            qs[r][c] = ok ? __ldg(Q + o) : 0.0f;
        }
        for (int i = threadIdx.x; i < AB_COLS * D; i += AB_THREADS) {
            const int c = i / D, j = i % D;
            gs[c][j] = (s0 + c < S) ? __ldg(dOut + (bh * S + s0 + c) * (int64_t)D + j) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int n = 0; n < 5; ++n) {
            if (ei[n] >= 0) {
                float a = accT[n], d = accD[n];
#pragma unroll 8
                for (int c = 0; c < AB_COLS; ++c) {
                    a = fmaf(ks[ei[n]][c], vs[ej[n]][c], a);
                    d = fmaf(qs[ei[n]][c], gs[c][ej[n]], d);
                }
                accT[n] = a; accD[n] = d;
            }
        }
    }
    float* w = ws + ((bh * chunks + chunk) * 2) * (int64_t)(AB_TP * AB_TP);
#pragma unroll
    for (int n = 0; n < 5; ++n)
        if (ei[n] >= 0) {
            w[ei[n] * AB_TP + ej[n]] = accT[n];
            w[AB_TP * AB_TP + ei[n] * AB_TP + ej[n]] = accD[n];
        }
}

__global__ void __launch_bounds__(128)
attn_bwd_apply_kernel(const float* __restrict__ K, const float* __restrict__ V, const float* __restrict__ dOut,
                      const float* __restrict__ ws, float* __restrict__ dQ, float* __restrict__ dK, float* __restrict__ dV,
                      int D, int S, int chunks, int col_tiles) {
    __shared__ float T[AB_MAXD][AB_TP], dT[AB_MAXD][AB_TP];
    __shared__ float gs[128][AB_TP + 1];
    const int64_t bh = blockIdx.x / col_tiles;
    const int s0 = (blockIdx.x % col_tiles) * 128;
    const float inv_s = 1.0f / (float)S;
    for (int e = threadIdx.x; e < D * D; e += blockDim.x) {
        const int i = e / D, j = e % D;
        float a = 0.0f, d = 0.0f;
        for (int c = 0; c < chunks; ++c) {
            const float* w = ws + ((bh * chunks + c) * 2) * (int64_t)(AB_TP * AB_TP);
            a += __ldg(w + i * AB_TP + j);
            d += __ldg(w + AB_TP * AB_TP + i * AB_TP + j);
        }
        T[i][j] = a * inv_s;
        dT[i][j] = d * inv_s;          // the 1/S of dK and dV folded in
    }
    for (int i = threadIdx.x; i < 128 * D; i += blockDim.x) {
        const int c = i / D, j = i % D;
        gs[c][j] = (s0 + c < S) ? __ldg(dOut + (bh * S + s0 + c) * (int64_t)D + j) : 0.0f;
    }
    __syncthreads();
    const int s = s0 + threadIdx.x;
    if (s >= S) return;
    const int64_t base = bh * (int64_t)D * S + s;
    float col[AB_MAXD];
    // dQ[i][s] = sum_j T[i][j] dOut[s][j]
    for (int i = 0; i < D; ++i) {
        float a = 0.0f;
        for (int j = 0; j < D; ++j) a = fmaf(T[i][j], gs[threadIdx.x][j], a);
        dQ[base + (int64_t)i * S] = a;
    }
    // dK[i][s] = sum_j dT[i][j] V[j][s]
    for (int j = 0; j < D; ++j) col[j] = __ldg(V + base + (int64_t)j * S);
    for (int i = 0; i < D; ++i) {
        float a = 0.0f;
        for (int j = 0; j < D; ++j) a = fmaf(dT[i][j], col[j], a);
        dK[base + (int64_t)i * S] = a;
    }
    // dV[j][s] = sum_i dT[i][j] K[i][s]
    for (int i = 0; i < D; ++i) col[i] = __ldg(K + base + (int64_t)i * S);
    for (int j = 0; j < D; ++j) {
        float a = 0.0f;
        for (int i = 0; i < D; ++i) a = fmaf(dT[i][j], col[i], a);
        dV[base + (int64_t)j * S] = a;
    }
}

static int attn_bwd_chunks(int64_t BH, int S) {
    const int tiles = ceil_div(S, AB_COLS);
    int64_t c = ceil_div((int64_t)num_sms() * 4, BH);
    if (c > tiles) c = tiles;
    if (c > 64) c = 64;
    if (c < 1) c = 1;
    return (int)c;
}

}  // namespace spgt

using namespace spgt;

extern "C" size_t spgt_galerkin_attn_bwd_workspace_bytes(int B, int H, int dpk, int S) {
    if (B <= 0 || H <= 0 || S <= 0 || dpk < 1 || dpk > AB_MAXD) return 0;
    return (size_t)B * H * attn_bwd_chunks((int64_t)B * H, S) * 2 * AB_TP * AB_TP * sizeof(float);
}

extern "C" int spgt_galerkin_attn_bwd(const float* Q, const float* K, const float* V, const float* d_out, float* dQ, float* dK,
                                      float* dV, int B, int H, int dpk, int S, void* workspace, size_t workspace_bytes,
                                      spgt_stream_t stream) {
    if (!Q || !K || !V || !d_out || !dQ || !dK || !dV) return SPGT_ERR_NULL;
    if (B <= 0 || H <= 0 || S <= 0 || dpk < 1 || dpk > AB_MAXD) return SPGT_ERR_SHAPE;
    const int64_t BH = (int64_t)B * H;
    const int chunks = attn_bwd_chunks(BH, S), col_tiles = ceil_div(S, 128);
    if (BH * chunks > 0x7fffffffLL || BH * col_tiles > 0x7fffffffLL) return SPGT_ERR_SHAPE;
    if (!workspace || workspace_bytes < spgt_galerkin_attn_bwd_workspace_bytes(B, H, dpk, S)) return SPGT_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    attn_bwd_reduce_kernel<<<(unsigned)(BH * chunks), AB_THREADS, 0, st>>>(Q, K, V, d_out, (float*)workspace, dpk, S, chunks);
    if (int e = launch_status()) return e;
    attn_bwd_apply_kernel<<<(unsigned)(BH * col_tiles), 128, 0, st>>>(K, V, d_out, (const float*)workspace, dQ, dK, dV, dpk, S,
                                                                      chunks, col_tiles);
    return launch_status();
}
