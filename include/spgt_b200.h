/*
 * spgt_b200 -- C ABI of the B200 (sm_100a) kernels behind the SpGT inference hot path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*,
 * i.e. a cudaStream_t; NULL = the legacy default stream), launches asynchronously on that
 * stream and returns 0 on success or a negative SPGT_ERR_* code.  Nothing here allocates,
 * frees or synchronises unless its comment says so; callers own every buffer.  All tensors
 * are dense fp32 (complex64 = interleaved float pairs) and must be 16-byte aligned at their
 * base.  "Reference" paths below are relative to the Bloonow/SpGT source tree.
 */
#ifndef SPGT_B200_H_
#define SPGT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPGT_OK 0
#define SPGT_ERR_NULL (-1)        /* a required pointer is NULL */
#define SPGT_ERR_SHAPE (-2)       /* a size is non-positive, too large, or a combination is not supported */
#define SPGT_ERR_ALIGN (-3)       /* a base pointer is not 16-byte aligned */
#define SPGT_ERR_WORKSPACE (-4)   /* workspace missing or smaller than the *_workspace_bytes() answer */
#define SPGT_ERR_LAUNCH (-5)      /* the CUDA runtime refused the launch; see spgt_last_cuda_error() */
#define SPGT_ERR_TOO_LARGE (-6)   /* the problem exceeds the fixed scratch of a *_noalloc entry point */
#define SPGT_ERR_NOT_CONVERGED (-7) /* an iterative solver stopped at its iteration limit; outputs hold the last iterate */

#define SPGT_ACT_NONE 0
#define SPGT_ACT_RELU 1
#define SPGT_ACT_SILU 2
#define SPGT_ACT_SILU2 3          /* SiLU applied twice, as the reference's UpScaler2D does */

typedef void* spgt_stream_t;

/* Human-readable text for an SPGT_ERR_* code; never NULL. */
const char* spgt_error_string(int code);
/* cudaError_t of the most recent failed launch in this thread (0 if none). */
int spgt_last_cuda_error(void);
/* Library ABI version (bumped when a signature changes). */
int spgt_abi_version(void);
/* Experiment knobs: "attn_cluster" = 0 (heuristic), 1, 2, 4 or 8 CTAs per (batch, head) in spgt_galerkin_attn_fwd;
 * "attn_impl" = 0 (tcgen05 kernel, default) or 1 (warp-MMA kernel);
 * "spectral_chunk_mb" = megabytes of x per chunk of the spectral layer (0 = whole batch, default). */
int spgt_set_tuning(const char* key, int value);

/* ---------------------------------------------------------------------------------------------
 * Galerkin attention ops (reference: extension/bind/galerkin_attention.{py,cu})
 * ------------------------------------------------------------------------------------------- */

/* out[b,h,d_pos+c,s] = sum_k x[b,s,k] * w[k,h*d_head+c] + bias[h*d_head+c];  out[b,h,0:d_pos,s] = pos[b,s,:].
 * x [B,S,D], w [D,D] (used as [k][n], NOT transposed), bias [D], pos [B,S,d_pos], out [B,H,d_pos+d_head,S].
 * Requires D == H*d_head, d_head == 32, D % 128 == 0, d_pos in [0,8].
 * Replaces multihead_projection_with_position_rrc_forward (extension/bind/galerkin_attention.cu:9-24)
 * -> mh32::sgemm_rrc_cuda (extension/native/multihead_dim32.cu:571-599). */
int spgt_projpos_fwd(const float* x, const float* w, const float* bias, const float* pos, float* out,
                     int B, int S, int D, int H, int d_head, int d_pos, spgt_stream_t stream);

/* Same projection followed by LayerNorm over the d_head channels of each (b,s,h) (biased variance,
 * y = (v-mu)*rsqrt(var+eps)*lnw[h,c]+lnb[h,c]); position rows are copied unnormalised.
 * invsigma [B,H,S] may be NULL (the reference saves it for its backward pass only).
 * Replaces multihead_projection_layernorm_with_position_rrc_forward
 * (extension/bind/galerkin_attention.cu:50-68; LayerNorm at extension/native/multihead_dim32.cu:59-146). */
int spgt_projpos_lnorm_fwd(const float* x, const float* w, const float* bias, const float* lnw, const float* lnb,
                           float eps, const float* pos, float* out, float* invsigma,
                           int B, int S, int D, int H, int d_head, int d_pos, spgt_stream_t stream);

/* One launch computing q, k, v of a self-attention layer from the same x (x is read once):
 * q = projpos(x, wq, bq), k = projpos_lnorm(x, wk, bk, lnwk, lnbk), v likewise.  Same shapes as above. */
int spgt_projpos_qkv_fwd(const float* x, const float* wq, const float* bq, const float* wk, const float* bk,
                         const float* wv, const float* bv, const float* lnwk, const float* lnbk,
                         const float* lnwv, const float* lnbv, float eps, const float* pos,
                         float* q, float* k, float* v, int B, int S, int D, int H, int d_head, int d_pos,
                         spgt_stream_t stream);

/* out[b,h,s,:] = Q[b,h,:,s]^T * T[b,h],  T[b,h,i,j] = (1/S) * sum_s K[b,h,i,s] * V[b,h,j,s].
 * Q,K,V [B*H, dpk, S]; out [B*H, S, dpk] when merged_heads == 0 (the reference layout), or
 * [B, S, H*dpk] when merged_heads != 0 (what the reference obtains with transpose(1,2).contiguous(),
 * network/sp_layer.py:74).  t_out [B*H, dpk, dpk] row-major (i,j) is optional (NULL to skip).
 * dpk must be in [32,35].  One thread-block cluster per (b,h) reduces T through distributed shared memory:
 * no global scratch, deterministic.  Replaces multihead_galerkin_attention_cccr_forward
 * (extension/bind/galerkin_attention.cu:104-124) = split-K SGEMM (extension/native/sgemm_32x32_splitk.cu:662-705)
 * + small-K SGEMM (extension/native/sgemm_32x32.cu:683-710). */
int spgt_galerkin_attn_fwd(const float* Q, const float* K, const float* V, float* out, float* t_out,
                           int B, int H, int dpk, int S, int merged_heads, spgt_stream_t stream);

/* Backward of spgt_galerkin_attn_fwd (not-merged output layout): gradients dQ, dK, dV [B,H,dpk,S] from d_out
 * [B,H,S,dpk].  Replaces multihead_galerkin_attention_cccr_backward (extension/bind/galerkin_attention.cu:126-173:
 * three split-K + three small-K SGEMMs) with one streaming reduction and one apply kernel in exact fp32 FMA
 * arithmetic; chunk partials are summed in chunk order (deterministic).  dpk <= 35. */
size_t spgt_galerkin_attn_bwd_workspace_bytes(int B, int H, int dpk, int S);
int spgt_galerkin_attn_bwd(const float* Q, const float* K, const float* V, const float* d_out, float* dQ, float* dK,
                           float* dV, int B, int H, int dpk, int S, void* workspace, size_t workspace_bytes,
                           spgt_stream_t stream);

/* Element-wise part of the backward of the projection (+ LayerNorm) + position op: from grad_out [B,H,d_pos+32,S] and the
 * pre-LayerNorm projection h = x W + b [B*S, H*32] it writes dh [B*S, H*32] (gradient with respect to h) and the parameter
 * gradients db, dlnw, dlnb [H*32] (dlnw, dlnb only with ln_weight != NULL; without LayerNorm dh is the gathered gradient
 * and h may be NULL).  The caller finishes with two GEMMs, dX = dh W^T and dW = x^T dh (spgt_linear_tc_fwd and
 * spgt_batched_transpose + spgt_batched_skinny_gemm).  Replaces the element-wise stages of
 * multihead_projection[_layernorm]_with_position_rrc_backward (extension/bind/galerkin_attention.cu:26-48, 70-102).
 * Partial sums are added in block order (deterministic).  d_head must be 32, H <= 8. */
size_t spgt_projpos_bwd_workspace_bytes(int B, int S, int H);
int spgt_projpos_bwd_elementwise(const float* grad_out, const float* h, const float* ln_weight, float eps, float* dh, float* db,
                                 float* dlnw, float* dlnb, int B, int S, int H, int d_head, int d_pos, void* workspace,
                                 size_t workspace_bytes, spgt_stream_t stream);

/* C[b] = alpha * A[b] * B[b] with A [batch,M,K], B [batch,K,N], C [batch,M,N], all row-major; K is the long
 * dimension.  N % 4 == 0: one launch of a persistent kernel that cuts the k range of all (batch, 32x32 tile) items
 * evenly over one CTA per SM; items that span several CTAs leave partial tiles (and a ticket count) in `workspace`
 * and the CTA that finishes last adds them in CTA order.  Other N: split-K in two passes with per-split partial
 * tiles in `workspace`, summed in split order.  Both are deterministic (bit-identical from run to run).
 * Replaces batched_skinny_gemm (extension/bind/galerkin_attention.cu:175-198, GEMM_Order::RRR). */
size_t spgt_skinny_gemm_workspace_bytes(int M, int N, int K, int batch);
int spgt_batched_skinny_gemm(const float* A, const float* B, float* C, float alpha, int M, int N, int K, int batch,
                             void* workspace, size_t workspace_bytes, spgt_stream_t stream);

/* The same product for callers that can neither pass a workspace nor allocate one (plugin callbacks, real-time
 * loops, hosts whose device allocator is out of reach at call time).  No counterpart in the reference, whose
 * binding allocates its split-K buffer through torch on every call.  The scratch (partial tiles and ticket
 * counts) lives in a fixed 8 MiB array inside the library image (one per device); the call allocates nothing and
 * runs the same kernels on the same plan as spgt_batched_skinny_gemm (bit-identical result).
 *  - Limit: spgt_skinny_gemm_workspace_bytes(M,N,K,batch) must not exceed spgt_skinny_gemm_noalloc_max_bytes();
 *    otherwise SPGT_ERR_TOO_LARGE is returned and nothing is launched.
 *  - The first call on each device (that device current) looks up the array's device address and sets kernel
 *    attributes; with lazy module loading it may also be the call that loads the module holding the array.  Make it
 *    before any stream capture.  Later calls only clear the ticket counts (a memset on the stream) and launch kernels.
 *  - The array keeps the last call's contents.  Partial tiles need no clearing (every tile that is read is written
 *    earlier in the same call); the ticket counts must start at zero and are cleared by each call.
 *  - One array per device: calls that may overlap on a device (different streams) race; keep them on one stream
 *    or order them with events. */
size_t spgt_skinny_gemm_noalloc_max_bytes(void);
int spgt_batched_skinny_gemm_noalloc(const float* A, const float* B, float* C, float alpha, int M, int N, int K,
                                     int batch, spgt_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Validation metric (reference: engine/metric.py:47-67, WeightedL2Loss2D with alpha = 0, beta = 1)
 * ------------------------------------------------------------------------------------------- */

/* per_sample[n] = sqrt( mean((pred[n] - target[n])^2) / (mean(target[n]^2) + eps) ) over n_per_sample elements of
 * each of the N samples (dense, sample-major).  The reference reduces these per-sample values with a mean ('L1'),
 * sqrt of the mean of squares ('L2') or max ('Linf'); that reduction over N numbers is left to the caller.
 * One block per sample, fixed summation order. */
int spgt_relative_l2_fwd(const float* pred, const float* target, float* per_sample, int N, int64_t n_per_sample,
                         float eps, spgt_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Data generation (reference: dataset/darcy_generate/Solve_GWF.m, MATLAB)
 * ------------------------------------------------------------------------------------------- */

/* Finite-volume Darcy solve of the reference's generator, for B coefficient fields at once, in float64:
 *   sum over the 4 neighbours n of (a[n] + a[i,j]) / 2 * (p[i,j] - p[n]) * (K-1)^2 = f[i,j]  on the interior nodes of the
 *   K x K node grid, p = 0 on the boundary                          (the matrix of Solve_GWF.m:16-35).
 * coef_nodes, f_nodes, p_nodes [B, K, K] float64 on the device (border values of f are ignored, the border of p is set
 * to 0).  The reference calls MATLAB's sparse direct solver (Solve_GWF.m:38); this is a Jacobi-preconditioned conjugate
 * gradient iteration with deterministic reductions, stopped when every sample has |r| <= rel_tol * |f| (checked every
 * check_every iterations, which synchronises the stream) or after max_iter iterations (SPGT_ERR_NOT_CONVERGED, the
 * last iterate is kept).  iters_out (one int) and relres_out ([B]) are HOST pointers and may be NULL. */
size_t spgt_darcy_fv_workspace_bytes(int B, int K);
int spgt_darcy_fv_solve(const double* coef_nodes, const double* f_nodes, double* p_nodes, int B, int K, int max_iter,
                        double rel_tol, int check_every, void* workspace, size_t workspace_bytes, int* iters_out,
                        double* relres_out, spgt_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Data-movement ops (reference: extension/bind/datamove.{py,cu}, extension/native/datamove.cu)
 * ------------------------------------------------------------------------------------------- */

/* dst[b,n,m] = src[b,m,n].  Replaces datamove::batched_transpose_cuda (extension/native/datamove.cu:92-99). */
int spgt_batched_transpose(const float* src, float* dst, int M, int N, int batch, spgt_stream_t stream);

/* src complex64 [dim,H_all,W_all]; out_k[h,w,c] = src[c,hb_k+h,wb_k+w] for the two blocks k = 1,2.
 * Replaces transpose_gather_dual (extension/bind/datamove.cu:25-44). */
int spgt_transpose_gather_dual(const float* src, float* out1, float* out2, int dim, int H_all, int W_all,
                               int H_low, int W_low, int hb1, int wb1, int hb2, int wb2, spgt_stream_t stream);

/* Inverse of the gather; every element of out [dim,H_all,W_all] outside the two blocks is written as 0
 * (the reference allocates the output with torch::zeros).  If the blocks overlap, block 2 wins.
 * Replaces transpose_scatter_dual (extension/bind/datamove.cu:46-64). */
int spgt_transpose_scatter_dual(const float* src1, const float* src2, float* out, int dim, int H_all, int W_all,
                                int H_low, int W_low, int hb1, int wb1, int hb2, int wb2, spgt_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Dense layers the reference leaves to cuBLAS / cuDNN / ATen (network/layer.py, network/model.py)
 * ------------------------------------------------------------------------------------------- */

/* y[r, 0:N] = act(x[r, 0:K] * w[0:K, 0:N] + bias) (+ residual[r, 0:N]); w is [K,N] row-major (= torch Linear
 * weight transposed) with row pitch ldw.  lda/ldw/ldc/ldr are row pitches in floats (lda, ldw, K multiples of 4).
 * bias, residual may be NULL.
 * Covers nn.Linear + activation + residual add: FeedForward (network/layer.py:165-174), fc_layer
 * (network/sp_layer.py:75), residual_layer (network/sp_layer.py:131). */
int spgt_linear_fwd(const float* x, int lda, const float* w, int ldw, const float* bias, const float* residual, int ldr,
                    float* y, int ldc, int rows, int K, int N, int act, spgt_stream_t stream);

/* 3x3 convolution, padding 1, NHWC.  x [B,Hh,Ww,cin_pitch] using channels [cin_off, cin_off+Cin);
 * w [9*Cin, Cout] with row index (ky*3+kx)*Cin+ci and row pitch ldw (multiple of 4);
 * y [B,Hh,Ww,cout_pitch] channels [cout_off, cout_off+Cout); y = act(conv + bias).
 * Cin, cin_off, cin_pitch must be even.
 * Covers ConvResBlock2D (network/layer.py:16-24) for conv1..3 of DownScaler2D and the UpScaler2D conv. */
int spgt_conv3x3_fwd(const float* x, int cin_pitch, int cin_off, int Cin, const float* w, int ldw, const float* bias,
                     float* y, int cout_pitch, int cout_off, int Cout, int B, int Hh, int Ww, int act,
                     spgt_stream_t stream);

/* Bilinear resize, align_corners=True, NHWC [B,Hi,Wi,C] -> [B,Ho,Wo,C], followed by act.  C % 4 == 0.
 * Source coordinates are computed in fp32 exactly as ATen does (scale = (in-1)/(out-1), src = scale*dst).
 * Covers F.interpolate in DownScaler2D / UpScaler2D (network/model.py:30,36,59,63). */
int spgt_bilinear_fwd(const float* x, float* y, int B, int Hi, int Wi, int Ho, int Wo, int C, int act,
                      spgt_stream_t stream);

/* Bilinear resize of the channel concatenation of three NHWC tensors that keep their own channel pitch p_k
 * (only the first c_k channels of each are used), followed by act; y [B,Ho,Wo,c1+c2+c3] dense.
 * Covers torch.concat + F.interpolate + activation at the end of DownScaler2D (network/model.py:35-37). */
int spgt_bilinear_concat3_fwd(const float* x1, const float* x2, const float* x3, int p1, int p2, int p3, int c1, int c2,
                              int c3, float* y, int B, int Hi, int Wi, int Ho, int Wo, int act, spgt_stream_t stream);

/* First stage of DownScaler2D fused: y = act(bilinear(act(conv3x3(node) + bias))) with a 1-channel input.
 * node [B,Hi,Wi], w [9,Cout] (row = ky*3+kx), bias [Cout], y [B,Ho,Wo,Cout]; the Cout-channel full-resolution
 * tensor is never materialised.  Cout % 4 == 0, Cout <= 512.  (network/model.py:29-31.) */
int spgt_conv0_down_fwd(const float* node, const float* w, const float* bias, float* y, int B, int Hi, int Wi,
                        int Ho, int Wo, int Cout, int act, spgt_stream_t stream);

/* Last stage of UpScaler2D fused with the decoder's spatial_fc_layer: because both the bilinear resize and
 * the Linear are linear maps, Linear(concat(resize(u), grid)) = resize(u * Wx) + grid * Wg + bias.
 * uw [B,Hi,Wi,C] already holds u * Wx; grid [B,Ho,Wo,2]; wg [2,C]; bias [C]; y [B,Ho,Wo,C].  C % 4 == 0.
 * (network/model.py:63-64, network/sp_model.py:59-60.) */
int spgt_upsample_grid_fwd(const float* uw, const float* grid, const float* wg, const float* bias, float* y,
                           int B, int Hi, int Wi, int Ho, int Wo, int C, spgt_stream_t stream);

/* Decoder FeedForward with a scalar target, de-normalisation and the Dirichlet frame in one pass:
 * out[b,y,x] = ((act(x*w1+b1) . w2) + b2) * scale + shift, then 0 on the 1-pixel frame if dirichlet != 0.
 * scale_map / shift_map [Hh*Ww] are optional per-pixel replacements of scale / shift (a normaliser fitted per
 * grid node); pass NULL to use the scalars.
 * x [B*Hh*Ww, K] (K % 4 == 0, K <= 64), w1 [K,N1] (N1 == 128), w2 [N1].
 * (network/sp_model.py:63, 109-112; dataset/darcy_dataset.py:30-31.) */
int spgt_decoder_head_fwd(const float* x, const float* w1, const float* b1, const float* w2, float b2,
                          float scale, float shift, const float* scale_map, const float* shift_map, int dirichlet,
                          float* out, int B, int Hh, int Ww, int K, int N1, int act, spgt_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * tcgen05 / TMEM variants of the dense layers (same math, 3xTF32 on the 5th-generation tensor cores).
 * Weights are prepared once: split into tf32 hi / lo planes, transposed to K-major [Npad][Kpad], zero padded.
 * No counterpart in the reference, which leaves these layers to cuBLAS / cuDNN.
 * ------------------------------------------------------------------------------------------- */

/* Bytes of a prepared weight for a [K,N] matrix, and the preparation itself (w_kn row-major, pitch ldw). */
size_t spgt_tc_weight_bytes(int K, int N);
int spgt_tc_weight_prepare(const float* w_kn, int ldw, int K, int N, void* out, size_t out_bytes, spgt_stream_t stream);
/* 0 if no tensor-core kernel gave up on a bounded wait since the last reset, else the code of the first one that did
 * (GEMM: 1..9; fused feed-forward: 21..34; attention: 101..109; spectral layer: 201..219).  Every wait inside these
 * kernels is bounded by two seconds of wall time; a kernel whose wait expires stops waiting, records the code and
 * returns with an incomplete output, so a host loop should read this at its synchronisation points and discard the
 * results when it is not 0.  Synchronises the device.  No counterpart in the reference (its kernels have no waits). */
int spgt_tc_status(void);
/* Clears the latched code (after the caller has dealt with it).  Synchronises the device. */
int spgt_tc_status_reset(void);
/* Self-test of the bounded wait: launches one warp that waits, for at most limit_us microseconds (1..100000), on a
 * barrier nothing arrives at.  The wait gives up, latches `code` (> 0) as spgt_tc_status() reports it and the kernel
 * returns; *returned_dev (device int) is set to 2 when the wait expired, 1 if it was satisfied.  Test infrastructure. */
int spgt_tc_selftest_wait_expiry(int code, int limit_us, int* returned_dev, spgt_stream_t stream);

/* As spgt_linear_fwd with wprep = spgt_tc_weight_prepare(w, ...). */
int spgt_linear_tc_fwd(const float* x, int lda, const void* wprep, const float* bias, const float* residual, int ldr,
                       float* y, int ldc, int rows, int K, int N, int act, spgt_stream_t stream);
/* y = act(x W1 + b1) W2 + b2 (+ residual) with x [rows, D = 128], W1 [128, 256], W2 [256, 128] prepared by
 * spgt_tc_weight_prepare: both GEMMs of FeedForward.forward (network/layer.py:155-174) in one kernel, the hidden
 * activations stay in tensor memory.  Only D = 128, Hd = 256 is supported (SPGT_ERR_SHAPE otherwise). */
int spgt_ffn_tc_fwd(const float* x, int lda, const void* w1prep, const float* b1, const void* w2prep, const float* b2,
                    const float* residual, int ldr, float* y, int ldc, int rows, int D, int Hd, int act, spgt_stream_t stream);

/* As spgt_conv3x3_fwd with a prepared [9*Cin, Cout] weight; Cin, cin_off, cin_pitch must be multiples of 4. */
int spgt_conv3x3_tc_fwd(const float* x, int cin_pitch, int cin_off, int Cin, const void* wprep, const float* bias,
                        float* y, int cout_pitch, int cout_off, int Cout, int B, int Hh, int Ww, int act,
                        spgt_stream_t stream);
/* As spgt_projpos_qkv_fwd for D == 128, H == 4; wprep_qkv is prepared from the [128, 384] matrix Wq | Wk | Wv. */
int spgt_projpos_qkv_tc_fwd(const float* x, const void* wprep_qkv, const float* bq, const float* bk, const float* bv,
                            const float* lnwk, const float* lnbk, const float* lnwv, const float* lnbv, float eps,
                            const float* pos, float* q, float* k, float* v, int B, int S, int D, int H, int d_head,
                            int d_pos, spgt_stream_t stream);
/* As spgt_decoder_head_fwd with a prepared w1. */
int spgt_decoder_head_tc_fwd(const float* x, const void* w1prep, const float* b1, const float* w2, float b2,
                             float scale, float shift, const float* scale_map, const float* shift_map, int dirichlet,
                             float* out, int B, int Hh, int Ww, int K, int N1, int act, spgt_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * FNO2d spectral layer (reference: Sp_SpectralConv2D.forward, network/sp_layer.py:125-156)
 * ------------------------------------------------------------------------------------------- */

/* y = act(irfft2(mix(rfft2(x)[two corner blocks of m x m modes])) + x*wr + br), computed as a mode-truncated DFT
 * (only the 2m x m retained modes are ever formed; r may be prime).
 * x, y [B,r,r,C] NHWC with C == 32; wr [C,C] (= residual_layer.weight transposed), br [C];
 * fw0, fw1 [m,m,C,C,2] (the SpGT fourier_weight layout); 1 <= m <= 16, 2m <= r.
 * tables: spgt_spectral_tables_bytes(r,m) bytes filled once by spgt_spectral_tables_init.
 * workspace: spgt_spectral_workspace_bytes(B,r,m,C) bytes of scratch (contents undefined afterwards).
 * The batch can be processed in chunks of spgt_spectral_chunk_samples(r) samples (tuning key "spectral_chunk_mb",
 * megabytes of x per chunk; 0 = the whole batch, the default) so that the second pass over a chunk's x is served by
 * the L2 cache; the scratch is sized for one chunk, so query it after setting the key.
 * Replaces batched_transpose + torch.fft.rfft2 + transpose_gather_dual + complex matmul + transpose_scatter_dual
 * + torch.fft.irfft2 + batched_transpose + residual Linear + activation. */
size_t spgt_spectral_tables_bytes(int r, int m);
int spgt_spectral_tables_init(void* tables, size_t tables_bytes, int r, int m, spgt_stream_t stream);
size_t spgt_spectral_workspace_bytes(int B, int r, int m, int C);
int spgt_spectral_chunk_samples(int r);
/* Kernels one spgt_spectral_conv2d_fwd call launches for these sizes (launch accounting of benchmarks). */
int spgt_spectral_launches(int B, int r, int m);
int spgt_spectral_conv2d_fwd(const float* x, const float* wr, const float* br, const float* fw0, const float* fw1,
                             const void* tables, void* workspace, size_t workspace_bytes, float* y,
                             int B, int r, int C, int m, int act, spgt_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SPGT_B200_H_ */
