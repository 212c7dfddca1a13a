// Shared device helpers for the sm_100a kernels: 3xTF32 splitting, warp-level tensor-core MMA,
// cp.async staging, thread-block-cluster / distributed-shared-memory access, host-side checks.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/spgt_b200.h"

namespace spgt {

// ---- host side ---------------------------------------------------------------------------------
extern thread_local int g_last_cuda_error;

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { g_last_cuda_error = (int)e; return SPGT_ERR_LAUNCH; }
    return SPGT_OK;
}
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
// Kernel attributes and device properties are per device: every cache below is indexed by the current device, so
// one process may drive several GPUs.
constexpr int SPGT_MAX_DEVICES = 64;
inline int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= SPGT_MAX_DEVICES) dev = 0;
    return dev;
}
inline int num_sms() {
    static int n[SPGT_MAX_DEVICES] = {};
    const int dev = current_device();
    if (n[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        n[dev] = v;
    }
    return n[dev];
}
// Opt-in to more than 48 KB of dynamic shared memory, once per (kernel, device); `state` is a static of the call site.
struct SmemOptIn { size_t bytes[SPGT_MAX_DEVICES] = {}; };
template <class K> inline int smem_opt_in(K kern, size_t bytes, SmemOptIn& state) {
    const int dev = current_device();
    if (bytes > state.bytes[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) { g_last_cuda_error = (int)e; (void)cudaGetLastError(); return SPGT_ERR_LAUNCH; }
        state.bytes[dev] = bytes;
    }
    return SPGT_OK;
}
template <typename T> __host__ __device__ constexpr T ceil_div(T a, T b) { return (a + b - 1) / b; }

// ---- 3xTF32 ---------------------------------------------------------------------------------------
// x = hi + lo with hi = tf32(x) (round to nearest, ties away) and lo = x - hi (exact in fp32; the tensor core reads
// its upper 19 bits).  a*b ~= hi_a*hi_b + hi_a*lo_b + lo_a*hi_b recovers fp32-level accuracy from three TF32 MMAs.
// The rounding is done with integer arithmetic on the bit pattern (add half an ulp of tf32 to the magnitude, clear
// the 13 low mantissa bits): cvt.rna.tf32.f32 gives the same bits but runs on the quarter-rate conversion pipe,
// which becomes the bottleneck of kernels that split every operand element.
__device__ __forceinline__ uint32_t tf32_rna_bits(float x) { return (__float_as_uint(x) + 0x1000u) & 0xffffe000u; }
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    hi = tf32_rna_bits(x);
    lo = __float_as_uint(x - __uint_as_float(hi));
}

// Same, with lo also rounded to tf32 (round to nearest) instead of being truncated by the tensor core: two more
// instructions, unbiased error; used where thousands of products are summed (the K^T V reduction over grid nodes).
__device__ __forceinline__ void split_tf32_rn(float x, uint32_t& hi, uint32_t& lo) {
    hi = tf32_rna_bits(x);
    lo = tf32_rna_bits(x - __uint_as_float(hi));
}

// D(16x8) += A(16x8, row) * B(8x8, col), TF32 inputs, fp32 accumulate.
// Fragment layout (g = lane/4, t = lane%4):  a0=(g,t) a1=(g+8,t) a2=(g,t+4) a3=(g+8,t+4);
// b0=(k=t,n=g) b1=(k=t+4,n=g);  c0=(g,2t) c1=(g,2t+1) c2=(g+8,2t) c3=(g+8,2t+1).
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void mma_3xtf32(float (&c)[4], const uint32_t (&ahi)[4], const uint32_t (&alo)[4],
                                           const uint32_t (&bhi)[2], const uint32_t (&blo)[2]) {
    mma_tf32(c, alo, bhi);
    mma_tf32(c, ahi, blo);
    mma_tf32(c, ahi, bhi);
}

// ---- cp.async (global -> shared without registers) ---------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Copies BYTES (4, 8 or 16) when pred, otherwise fills the destination with zeros.  src must stay a valid
// address even when pred is false (it is not dereferenced: src-size 0).
template <int BYTES>
__device__ __forceinline__ void cp_async_zfill(void* smem_dst, const void* gsrc, bool pred) {
    const uint32_t d = smem_u32(smem_dst);
    const int n = pred ? BYTES : 0;
    if constexpr (BYTES == 16) {
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
    } else {
        asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(d), "l"(gsrc), "n"(BYTES), "r"(n) : "memory");
    }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- thread-block clusters -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// All threads of all CTAs of the cluster arrive, then wait: orders shared-memory writes before it against
// distributed-shared-memory reads after it.  This is a hardware barrier, not a spin on memory.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Read one float from the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ float ld_dsmem_f32(const float* local_smem_ptr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_smem_ptr)), "r"(rank));
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// ---- activations ---------------------------------------------------------------------------------------------
// x * sigmoid(x) with the hardware exp2 / reciprocal approximations: relative error below 1e-6, far inside the
// 1e-5 per-layer budget, at ~6 instructions instead of ~40 (the activation epilogues evaluate it 10^8 times).
__device__ __forceinline__ float silu_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
__device__ __forceinline__ float apply_act(float x, int act) {
    switch (act) {
        case SPGT_ACT_RELU: return fmaxf(x, 0.0f);
        case SPGT_ACT_SILU: return silu_f(x);
        case SPGT_ACT_SILU2: return silu_f(silu_f(x));
        default: return x;
    }
}

}  // namespace spgt
