// Finite-volume Darcy solve of the reference's data generator (dataset/darcy_generate/Solve_GWF.m:16-38):
//   sum over the four neighbours n of (a[n] + a[i,j]) / 2 * (p[i,j] - p[n]) * (K-1)^2 = f[i,j]   on the interior nodes of a
//   K x K grid, p = 0 on the boundary,
// for a batch of coefficient fields, by a Jacobi-preconditioned conjugate-gradient iteration in float64 (the
// reference solves the same symmetric positive definite system with MATLAB's sparse direct solver).
//
// HBM-bound streaming kernels, two per iteration over the whole batch:
//   step A   p <- z + beta p (neighbours too, from the previous p: ping-pong buffers), q = A p, partial sums of p.q
//   step B   alpha = (r.z) / (p.q); x += alpha p; r -= alpha q; z = r / diag(A); partial sums of r.z and r.r
// Every dot product is reduced in two fixed-order stages (per block, then over the blocks of a sample by every block
// that needs it), so results do not depend on scheduling.  All vectors are stored as full K x K grids whose border
// stays zero, which removes every boundary branch from the stencil.
#include <cmath>
#include <vector>

#include "common.cuh"

namespace spgt {

constexpr int DS_THREADS = 256;
constexpr int DS_NPT = 4;             // nodes per thread: amortises the per-block reduction of the previous step's partial sums

struct DsDims { int K, n, nblk; int64_t grid; };     // n = K - 2 interior nodes per side, nblk blocks per sample

__device__ __forceinline__ double ds_block_sum(double v, double* red) {
    // fixed-order tree over the block: lanes by shuffle, then warp 0 over the 8 warp sums
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double s = 0.0;
    if (threadIdx.x < 32) {
        s = threadIdx.x < DS_THREADS / 32 ? red[threadIdx.x] : 0.0;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) s += __shfl_down_sync(0xffffffffu, s, o);
    }
    return s;                                                    // valid in thread 0
}
// Sum of a sample's per-block partials, identical in every block that calls it.
__device__ __forceinline__ double ds_sample_sum(const double* part, int nblk, double* red) {
    double v = 0.0;
    for (int i = threadIdx.x; i < nblk; i += DS_THREADS) v += part[i];
    double s = ds_block_sum(v, red);
    __syncthreads();
    if (threadIdx.x == 0) red[8] = s;
    __syncthreads();
    return red[8];
}
__device__ __forceinline__ double ds_diag(const double* a, int K, double c) {
    return (a[-K] + a[K] + a[-1] + a[1] + 4.0 * c) * 0.5;
}

// x = 0, r = f, z = r / diag, p buffers = 0; partial sums of r.z and r.r (the latter is |b|^2 at this point)
__global__ void __launch_bounds__(DS_THREADS)
ds_init_kernel(const double* __restrict__ coef, const double* __restrict__ f, double* __restrict__ x, double* __restrict__ r,
               double* __restrict__ z, double* __restrict__ part_rz, double* __restrict__ part_rr, DsDims d) {
    __shared__ double red[9];
    const int b = blockIdx.y;
    const int64_t base = (int64_t)b * d.grid;
    double rz = 0.0, rr = 0.0;
#pragma unroll
    for (int k = 0; k < DS_NPT; ++k) {
        const int idx = (blockIdx.x * DS_NPT + k) * DS_THREADS + threadIdx.x;
        if (idx < d.n * d.n) {
            const int i = idx / d.n + 1, j = idx - (i - 1) * d.n + 1;
            const int64_t o = base + (int64_t)i * d.K + j;
            const double scale = (double)(d.K - 1) * (double)(d.K - 1);
            const double c = coef[o];
            const double rv = f[o], zv = rv / (ds_diag(coef + o, d.K, c) * scale);
            x[o] = 0.0; r[o] = rv; z[o] = zv;
            rz += rv * zv; rr += rv * rv;
        }
    }
    const double s1 = ds_block_sum(rz, red);
    const double s2 = ds_block_sum(rr, red);
    if (threadIdx.x == 0) { part_rz[(int64_t)b * d.nblk + blockIdx.x] = s1; part_rr[(int64_t)b * d.nblk + blockIdx.x] = s2; }
}

__global__ void __launch_bounds__(DS_THREADS)
ds_step_a_kernel(const double* __restrict__ coef, const double* __restrict__ z, const double* __restrict__ p_old,
                 double* __restrict__ p_new, double* __restrict__ q, const double* __restrict__ part_rz,
                 double* __restrict__ rz_hist, double* __restrict__ part_pq, int iter, DsDims d) {
    __shared__ double red[9];
    const int b = blockIdx.y;
    const double rz = ds_sample_sum(part_rz + (int64_t)b * d.nblk, d.nblk, red);
    double beta = 0.0;
    if (iter > 0) { const double prev = rz_hist[2 * b + ((iter - 1) & 1)]; beta = prev != 0.0 ? rz / prev : 0.0; }
    if (blockIdx.x == 0 && threadIdx.x == 0) rz_hist[2 * b + (iter & 1)] = rz;
    const int64_t base = (int64_t)b * d.grid;
    double pq = 0.0;
#pragma unroll
    for (int k = 0; k < DS_NPT; ++k) {
        const int idx = (blockIdx.x * DS_NPT + k) * DS_THREADS + threadIdx.x;
        if (idx < d.n * d.n) {
            const int i = idx / d.n + 1, j = idx - (i - 1) * d.n + 1;
            const int64_t o = base + (int64_t)i * d.K + j;
            const int K = d.K;
            const double scale = (double)(K - 1) * (double)(K - 1);
            // the new search direction at this node and at its four neighbours (border nodes: z = p = 0)
            const double pc = z[o] + beta * p_old[o];
            const double pn = z[o - K] + beta * p_old[o - K], ps = z[o + K] + beta * p_old[o + K];
            const double pw = z[o - 1] + beta * p_old[o - 1], pe = z[o + 1] + beta * p_old[o + 1];
            const double c = coef[o];
            const double wn = (coef[o - K] + c) * 0.5, ws = (coef[o + K] + c) * 0.5;
            const double ww = (coef[o - 1] + c) * 0.5, we = (coef[o + 1] + c) * 0.5;
            const double qv = (wn * (pc - pn) + ws * (pc - ps) + ww * (pc - pw) + we * (pc - pe)) * scale;
            p_new[o] = pc;
            q[o] = qv;
            pq += pc * qv;
        }
    }
    const double s = ds_block_sum(pq, red);
    if (threadIdx.x == 0) part_pq[(int64_t)b * d.nblk + blockIdx.x] = s;
}

__global__ void __launch_bounds__(DS_THREADS)
ds_step_b_kernel(const double* __restrict__ coef, const double* __restrict__ p, const double* __restrict__ q,
                 double* __restrict__ x, double* __restrict__ r, double* __restrict__ z, const double* __restrict__ part_pq,
                 const double* __restrict__ rz_hist, double* __restrict__ part_rz, double* __restrict__ part_rr, int iter,
                 DsDims d) {
    __shared__ double red[9];
    const int b = blockIdx.y;
    const double pq = ds_sample_sum(part_pq + (int64_t)b * d.nblk, d.nblk, red);
    const double alpha = pq != 0.0 ? rz_hist[2 * b + (iter & 1)] / pq : 0.0;
    const int64_t base = (int64_t)b * d.grid;
    double rz = 0.0, rr = 0.0;
#pragma unroll
    for (int k = 0; k < DS_NPT; ++k) {
        const int idx = (blockIdx.x * DS_NPT + k) * DS_THREADS + threadIdx.x;
        if (idx < d.n * d.n) {
            const int i = idx / d.n + 1, j = idx - (i - 1) * d.n + 1;
            const int64_t o = base + (int64_t)i * d.K + j;
            const double scale = (double)(d.K - 1) * (double)(d.K - 1);
            x[o] += alpha * p[o];
            const double rv = r[o] - alpha * q[o];
            const double zv = rv / (ds_diag(coef + o, d.K, coef[o]) * scale);
            r[o] = rv; z[o] = zv;
            rz += rv * zv; rr += rv * rv;
        }
    }
    const double s1 = ds_block_sum(rz, red);
    const double s2 = ds_block_sum(rr, red);
    if (threadIdx.x == 0) { part_rz[(int64_t)b * d.nblk + blockIdx.x] = s1; part_rr[(int64_t)b * d.nblk + blockIdx.x] = s2; }
}

static DsDims ds_dims(int K) {
    DsDims d; d.K = K; d.n = K - 2; d.nblk = ceil_div(d.n * d.n, DS_THREADS * DS_NPT); d.grid = (int64_t)K * K; return d;
}
static size_t ds_align(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace spgt

using namespace spgt;

extern "C" size_t spgt_darcy_fv_workspace_bytes(int B, int K) {
    if (B <= 0 || K < 3) return 0;
    const DsDims d = ds_dims(K);
    const size_t vec = ds_align((size_t)B * d.grid * sizeof(double));
    const size_t part = ds_align((size_t)B * d.nblk * sizeof(double));
    return 5 * vec + 3 * part + ds_align((size_t)2 * B * sizeof(double));
}

extern "C" int spgt_darcy_fv_solve(const double* coef_nodes, const double* f_nodes, double* p_nodes, int B, int K, int max_iter,
                                   double rel_tol, int check_every, void* workspace, size_t workspace_bytes, int* iters_out,
                                   double* relres_out, spgt_stream_t stream) {
    if (!coef_nodes || !f_nodes || !p_nodes || !workspace) return SPGT_ERR_NULL;
    if (B <= 0 || K < 3 || K > 8192 || max_iter <= 0 || check_every <= 0 || !(rel_tol > 0.0)) return SPGT_ERR_SHAPE;
    if (workspace_bytes < spgt_darcy_fv_workspace_bytes(B, K)) return SPGT_ERR_WORKSPACE;
    if (!aligned16(coef_nodes) || !aligned16(f_nodes) || !aligned16(p_nodes) || !aligned16(workspace)) return SPGT_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    const DsDims d = ds_dims(K);
    const size_t vec = ds_align((size_t)B * d.grid * sizeof(double));
    const size_t part = ds_align((size_t)B * d.nblk * sizeof(double));
    uint8_t* w = (uint8_t*)workspace;
    double* r = (double*)w; double* z = (double*)(w + vec); double* p0 = (double*)(w + 2 * vec); double* p1 = (double*)(w + 3 * vec);
    double* q = (double*)(w + 4 * vec);
    double* part_rz = (double*)(w + 5 * vec); double* part_rr = (double*)(w + 5 * vec + part); double* part_pq = (double*)(w + 5 * vec + 2 * part);
    double* rz_hist = (double*)(w + 5 * vec + 3 * part);
    // borders of every vector (and the whole first search direction) must be zero
    if (cudaMemsetAsync(workspace, 0, 5 * vec, st) != cudaSuccess) return launch_status();
    if (cudaMemsetAsync(p_nodes, 0, (size_t)B * d.grid * sizeof(double), st) != cudaSuccess) return launch_status();
    const dim3 grid(d.nblk, B);
    ds_init_kernel<<<grid, DS_THREADS, 0, st>>>(coef_nodes, f_nodes, p_nodes, r, z, part_rz, part_rr, d);
    if (int e = launch_status()) return e;

    std::vector<double> host_rr((size_t)B * d.nblk), bnorm2(B, 0.0), rel(B, 0.0);
    auto residuals = [&](std::vector<double>& out) -> int {
        if (cudaMemcpyAsync(host_rr.data(), part_rr, host_rr.size() * sizeof(double), cudaMemcpyDeviceToHost, st) != cudaSuccess) return SPGT_ERR_LAUNCH;
        if (cudaStreamSynchronize(st) != cudaSuccess) return SPGT_ERR_LAUNCH;
        for (int b = 0; b < B; ++b) {
            double s = 0.0;
            for (int i = 0; i < d.nblk; ++i) s += host_rr[(size_t)b * d.nblk + i];
            out[b] = s;
        }
        return SPGT_OK;
    };
    if (int e = residuals(bnorm2)) return e;
    int it = 0;
    bool done = false;
    while (it < max_iter && !done) {
        const int stop = it + check_every < max_iter ? it + check_every : max_iter;
        for (; it < stop; ++it) {
            double* po = (it & 1) ? p1 : p0;
            double* pn = (it & 1) ? p0 : p1;
            ds_step_a_kernel<<<grid, DS_THREADS, 0, st>>>(coef_nodes, z, po, pn, q, part_rz, rz_hist, part_pq, it, d);
            ds_step_b_kernel<<<grid, DS_THREADS, 0, st>>>(coef_nodes, pn, q, p_nodes, r, z, part_pq, rz_hist, part_rz, part_rr, it, d);
        }
        if (int e = launch_status()) return e;
        if (int e = residuals(rel)) return e;
        done = true;
        for (int b = 0; b < B; ++b) {
            rel[b] = bnorm2[b] > 0.0 ? sqrt(rel[b] / bnorm2[b]) : 0.0;
            if (!(rel[b] <= rel_tol)) done = false;
        }
    }
    if (iters_out) *iters_out = it;
    if (relres_out) for (int b = 0; b < B; ++b) relres_out[b] = rel[b];
    return done ? SPGT_OK : SPGT_ERR_NOT_CONVERGED;
}
