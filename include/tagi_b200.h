/* tagi_b200.h - C ABI of the B200 (sm_100a) TAGI Linear / Conv2d hot path.
 *
 * Every entry point takes plain pointers and sizes, returns an int status
 * (TAGI_OK = 0) and never exits or throws; tagi_last_error_string() gives the
 * reason for the last non-zero status on the calling thread. Unless an entry
 * point says "host", pointers are DEVICE pointers owned by the caller, `stream`
 * is a cudaStream_t passed as void* (NULL = the legacy default stream, which
 * is what the reference's launchers use) and the call is asynchronous.
 * Inputs and outputs of one call must not alias. Outputs are fully overwritten
 * for the live extent (B x features) and nothing beyond it is touched.
 *
 * Layouts (row-major, flat FP32, as in the reference):
 *   activations / deltas  [B][features]        (src/linear_layer.cpp:44-54)
 *   Linear weights        [N][K]               (src/linear_layer.cpp:46)
 *   conv activations      [B][C][H][W], weights [fo][fi][k][k],
 *   conv outputs          [B][fo][ho*wo]       (src/conv2d_layer.cpp:297-314)
 *
 * File:line citations name the reference interface that each entry point
 * replaces (paths inside the cuTAGI source tree).
 */
#ifndef TAGI_B200_H
#define TAGI_B200_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

enum {
    TAGI_OK = 0,
    TAGI_ERR_INVALID_ARGUMENT = 1, /* null pointer, non-positive size, misaligned pointer, bad geometry */
    TAGI_ERR_CUDA = 2,             /* a CUDA runtime / driver call failed */
    TAGI_ERR_UNSUPPORTED = 3,      /* requested implementation cannot run this shape */
    TAGI_ERR_COMM = 4              /* NCCL / rendezvous failure */
};

/* Which arithmetic the Linear and Conv2d entry points use.
 *   AUTO   : the measured-faster variant that supports the shape (default)
 *   FFMA   : FP32 fused multiply-add on the CUDA cores, any shape
 *   TF32X3 : tcgen05 tensor-core MMA, each FP32 product split into three TF32 products
 *            (hi*hi + hi*lo + lo*hi) accumulated in FP32 in tensor memory;
 *            shapes it cannot run return TAGI_ERR_UNSUPPORTED under this setting. Conv2d runs on the same kernels
 *            after a gather pass that lays the receptive fields out as a matrix in library-owned scratch memory. */
enum { TAGI_IMPL_AUTO = 0, TAGI_IMPL_FFMA = 1, TAGI_IMPL_TF32X3 = 2 };
/* activations that tagi_linear_fwd_act / tagi_conv2d_fwd_act can fold into the forward pass */
enum { TAGI_ACT_RELU = 1, TAGI_ACT_MIXTURE_RELU = 2 };
int tagi_set_impl(int impl);
int tagi_get_impl(void);

/* Diagnostics of the TF32X3 kernels. Their device-side waits (on TMA and MMA completion barriers) are bounded; a wait
 * that runs out makes the kernel stop, release its tensor memory and record a non-zero code here instead of hanging.
 * tagi_tc_status copies the current device's status word to *status (0 = no wait ever ran out) and clears it when
 * `reset` is non-zero; it synchronises with the device. */
int tagi_tc_status(int *status, int reset);
/* Diagnostic switch of the TF32X3 kernels. on != 0 (default): the contraction is accumulated in tensor memory in
 * chunks of 256 that are summed in FP32 registers, which keeps the tensor core's accumulation error far below the
 * 1e-5 / 1e-4 tolerance. on == 0: one accumulation chain over the whole contraction (less accurate; for measurement). */
int tagi_tc_set_chunked(int on);
/* Diagnostic switch of the TF32X3 kernels. 3 (default): CTA pairs (tcgen05 cta_group::2, 256-row tiles, A-side operand
 * tiles in tensor memory, each CTA stages half of the B rows; passes with fewer than 256 output rows use the one-CTA
 * kernel); 1: one CTA per 128-row tile for every pass; 64, 80, 96, 112 or 128: as 3 with that tile width. Same results
 * in all of them. Process-wide like the other switches here (tagi_set_impl, tagi_tc_set_chunked, tagi_tc_set_sm_budget):
 * each is one atomic word, read when a kernel launch is planned, so a change from another host thread takes effect for
 * the launches planned after it (an entry point that launches several kernels may see it between two of them). */
int tagi_tc_set_variant(int v);
/* How many SMs the TF32X3 kernels plan their tile widths for: 0 (default) = all 148. A caller that runs another kernel
 * next to them (the data-parallel exchange's NCCL kernels on their own stream hold some SMs for the length of a pass)
 * passes the number that is left, so that a pass is cut into whole waves of the SMs it really gets: with 8 SMs taken,
 * 148 tiles would need three waves of 70 pairs where 128 wider tiles need two. Results do not depend on it. No
 * counterpart in the reference. */
int tagi_tc_set_sm_budget(int sms);

/* Library-owned scratch memory. The Conv2d entry points (regrouped weights, partial sums of a split contraction, the
 * operand matrices of the layers that still gather through memory) and tagi_bn2d_* (per-slice statistics) keep their
 * temporaries in one block per device that grows on demand with cudaMalloc. A block that was handed out is never freed
 * behind the caller's back: when a larger one is needed the old block is kept until tagi_release_scratch, so kernels in
 * flight and CUDA graphs captured earlier stay valid. Growth is refused (TAGI_ERR_UNSUPPORTED) while the call's stream
 * is being captured. To keep every allocation out of the training loop, size the block up front:
 *   tagi_conv2d_workspace_bytes(g)  bytes the three Conv2d passes of geometry g can ask for (host, no CUDA call);
 *   tagi_reserve_scratch(bytes)     make the current device's block at least that large (allocates; call at set-up);
 *   tagi_release_scratch()          synchronise the current device and free its block and every retired one;
 *   tagi_scratch_bytes()            size of the current device's block (host, no CUDA call besides cudaGetDevice).
 * Rules: calls that use scratch on one device must be ordered on the GPU (one stream, or events between streams), and
 * only one host thread at a time may issue such calls for a device: the block's contents are not protected. The
 * reference gives its launchers caller-owned temp_states.tmp_1 / tmp_2 for the same purpose
 * (src/conv2d_layer_cuda.cu:90-227); no counterpart for the three calls themselves. */
struct tagi_conv2d_geom;
size_t tagi_conv2d_workspace_bytes(const struct tagi_conv2d_geom *g);
int tagi_reserve_scratch(size_t bytes);
int tagi_release_scratch(void);
size_t tagi_scratch_bytes(void);

const char *tagi_last_error_string(void);
/* Library version as major*10000 + minor*100 + patch. */
int tagi_version(void);

/* ------------------------------------------------------------------ Linear */

/* mu_z = mu_a.mu_w^T + mu_b ; var_z = var_a.(mu_w^2+var_w)^T + mu_a^2.var_w^T + var_b.
 * Replaces linear_forward_cuda (src/linear_layer_cuda.cu:12-73) and its kernels
 * linear_fwd_mean_var_v4/v3/v1 (include/linear_cuda_kernel.cuh:375,246,50); the CPU definition is
 * linear_fwd_mean_var (src/linear_layer.cpp:10-60). mu_b/var_b may be NULL when has_bias == 0. */
int tagi_linear_fwd(const float *mu_w, const float *var_w, const float *mu_b, const float *var_b,
                    const float *mu_a, const float *var_a, int B, int K, int N, int has_bias,
                    float *mu_z, float *var_z, void *stream);

/* dmu_a = jcb * (dmu_z.mu_w) ; dvar_a = jcb^2 * (dvar_z.mu_w^2).
 * Replaces linear_state_backward_cuda (src/linear_layer_cuda.cu:75-121), kernels linear_bwd_delta_z_v4/v3
 * (include/linear_cuda_kernel.cuh:894,776); CPU definition linear_bwd_fc_delta_z (src/linear_layer.cpp:245-272).
 * jcb is the Jacobian saved by the forward pass (bwd_states->jcb), [B][K]; NULL stands for a Jacobian of ones (the
 * input of the layer was not an activation's output: cuTAGI fills bwd_states->jcb with ones then,
 * src/base_layer_cuda.cu:464-486), which saves reading it. */
int tagi_linear_bwd_state(const float *mu_w, const float *jcb, const float *dmu_z, const float *dvar_z,
                          int B, int K, int N, float *dmu_a, float *dvar_a, void *stream);

/* dmu_w = var_w * (dmu_z^T.mu_a) ; dvar_w = var_w^2 * (dvar_z^T.mu_a^2) ;
 * dmu_b = var_b * sum_b dmu_z ; dvar_b = var_b^2 * sum_b dvar_z  (bias part only when has_bias != 0).
 * Replaces linear_weight_backward_cuda (src/linear_layer_cuda.cu:123-168), kernels linear_bwd_delta_w_v4/v3
 * (include/linear_cuda_kernel.cuh:1320,1200) and the linear_bwd_delta_b launch (src/linear_layer_cuda.cu:311-321);
 * CPU definitions linear_bwd_fc_delta_w / _delta_b (src/linear_layer.cpp:314-349, 391-423).
 * mu_a is the input mean saved by the forward pass (bwd_states->mu_a), [B][K]. */
int tagi_linear_bwd_param(const float *var_w, const float *var_b, const float *mu_a, const float *dmu_z,
                          const float *dvar_z, int B, int K, int N, int has_bias, float *dmu_w, float *dvar_w,
                          float *dmu_b, float *dvar_b, void *stream);

/* The same pass for the output features n0 .. n1-1 only: rows n0 .. n1-1 of dmu_w / dvar_w and entries n0 .. n1-1 of
 * dmu_b / dvar_b are written, everything else is left alone. All pointers are those of the whole tensors. A caller that
 * exchanges the deltas between data-parallel ranks in pieces (src/ddp.cpp:113-146 exchanges whole tensors after the
 * whole backward pass) runs the pass range by range and starts the exchange of a range while the next one is computed;
 * the ranges together give exactly the result of tagi_linear_bwd_param. */
int tagi_linear_bwd_param_rows(const float *var_w, const float *var_b, const float *mu_a, const float *dmu_z,
                               const float *dvar_z, int B, int K, int N, int n0, int n1, int has_bias, float *dmu_w,
                               float *dvar_w, float *dmu_b, float *dvar_b, void *stream);

/* ------------------------------------------------------------------ Conv2d */

/* Geometry of one Conv2d call. The receptive field of output pixel (oy, ox), tap (ky, kx) is input pixel
 * (oy*stride - off + ky, ox*stride - off + kx), off = pad for pad_type 1, off = 0 (padding on the bottom / right
 * only) for pad_type 2 and for no padding; taps outside the image contribute nothing (src/indices.cpp:63-104,
 * 163-194; src/conv2d_layer.cpp:299). ho / wo must equal tagi_conv2d_out_size()'s result. No index tables and
 * no temporary buffers are needed: the kernels compute the gather arithmetically. */
typedef struct tagi_conv2d_geom {
    int B, fi, hi, wi, fo, ho, wo, k, stride, pad, pad_type, has_bias;
} tagi_conv2d_geom;

/* Host helper. Output extent by the reference's rule (compute_downsample_img_size_v2, src/conv2d_layer.cpp:581-628):
 * pad_type 1: (w - k + 2*pad)/stride + 1 ; 2: (w - k + pad)/stride + 1 ; else (w - k)/stride + 1.
 * TAGI_ERR_INVALID_ARGUMENT where the reference raises (numerator not divisible by the stride). */
int tagi_conv2d_out_size(int k, int stride, int wi, int hi, int pad, int pad_type, int *wo, int *ho);

/* Replaces conv2d_forward_cuda (src/conv2d_layer_cuda.cu:22-88), kernels conv2d_fwd_mean_var_cuda_v3/v2/v1
 * (include/conv2d_cuda_kernel.cuh:491,351,260); CPU definition conv2d_fwd_mean_var (src/conv2d_layer.cpp:274-322). */
int tagi_conv2d_fwd(const tagi_conv2d_geom *g, const float *mu_w, const float *var_w, const float *mu_b,
                    const float *var_b, const float *mu_a, const float *var_a, float *mu_z, float *var_z,
                    void *stream);

/* Replaces conv2d_state_backward_cuda (src/conv2d_layer_cuda.cu:90-147), kernels conv2d_bwd_delta_z_cuda_v2/v1
 * (include/conv2d_cuda_kernel.cuh:948,864) and the Jacobian permute launch (src/conv2d_layer_cuda.cu:504-511);
 * CPU definition conv2d_bwd_delta_z (src/conv2d_layer.cpp:363-403). jcb is in the natural [B][fi][hi*wi] layout; NULL
 * stands for a Jacobian of ones, as for tagi_linear_bwd_state. */
int tagi_conv2d_bwd_state(const tagi_conv2d_geom *g, const float *mu_w, const float *jcb, const float *dmu_z,
                          const float *dvar_z, float *dmu_a, float *dvar_a, void *stream);

/* Replaces conv2d_param_backward_cuda (src/conv2d_layer_cuda.cu:149-227), kernels conv2d_bwd_delta_w_cuda_v3/v2/v1
 * (include/conv2d_cuda_kernel.cuh:1333,1199,1109), permute_delta_cuda (:241) and the bias reduction
 * conv2d_bwd_delta_b_dual_sum_reduction (include/conv2d_cuda_kernel.cuh:812-860); CPU definitions conv2d_bwd_delta_w /
 * _delta_b (src/conv2d_layer.cpp:459-494, 538-556). Deltas are in the natural [B][fo][ho*wo] layout. */
int tagi_conv2d_bwd_param(const tagi_conv2d_geom *g, const float *var_w, const float *var_b, const float *mu_a,
                          const float *dmu_z, const float *dvar_z, float *dmu_w, float *dvar_w, float *dmu_b,
                          float *dvar_b, void *stream);

/* ------------------------------------------------------------------ neighbours of the path
 * Elementwise steps that sit between the calls above in a TAGI training step. They are memory-bound and outside the
 * hot path; they are here so that whole steps can run on the device through this library alone. */

/* ReLU moments: mu_a = max(mu_z, 0); where that is 0: jcb = 0, var_a = 0, else jcb = 1, var_a = var_z.
 * CPU definition relu_mean_var (src/activation.cpp:7-29); replaces relu_mean_var_cuda (src/activation_cuda.cu:8-24).
 * This call and tagi_mixture_relu_fwd may run in place: mu_a may be mu_z and var_a may be var_z (jcb must be distinct). */
int tagi_relu_fwd(const float *mu_z, const float *var_z, size_t n, float *mu_a, float *var_a, float *jcb, void *stream);

/* tagi_linear_fwd / tagi_conv2d_fwd followed by tagi_relu_fwd on their outputs, as one call: mu_a_out, var_a_out and
 * jcb_out are what the ReLU layer behind the Linear / Conv2d layer would hold; the moments before the ReLU are not
 * written. Where the forward pass runs on CTA pairs (256 or more output rows) the ReLU is applied in the kernel's
 * epilogue, which saves the ReLU pass's reads and the write of the pre-activation moments; otherwise the two steps run
 * one after the other. Results are those of the two separate calls, bit for bit. Replaces LinearCuda::forward /
 * Conv2dCuda::forward followed by ReLUCuda::forward -> relu_mean_var_cuda (src/activation_cuda.cu:8-24, 510-544) when a
 * ReLU layer follows the layer directly; nothing else reads the layer's own output. */
int tagi_linear_fwd_relu(const float *mu_w, const float *var_w, const float *mu_b, const float *var_b, const float *mu_a,
                         const float *var_a, int B, int K, int N, int has_bias, float *mu_a_out, float *var_a_out,
                         float *jcb_out, void *stream);
/* The same with the activation named by `act`: TAGI_ACT_RELU, or TAGI_ACT_MIXTURE_RELU for tagi_mixture_relu_fwd's
 * moments (MixtureReLUCuda::forward -> mixture_relu_mean_var_cuda, src/activation_cuda.cu:130-157, 726-759). Only the ReLU
 * runs inside the forward kernel; the MixtureReLU always runs as a second step in place on the outputs (its erf / exp
 * arithmetic in the epilogue was measured slower than a pass of its own). */
int tagi_linear_fwd_act(const float *mu_w, const float *var_w, const float *mu_b, const float *var_b, const float *mu_a,
                        const float *var_a, int B, int K, int N, int has_bias, int act, float *mu_a_out, float *var_a_out,
                        float *jcb_out, void *stream);
int tagi_conv2d_fwd_act(const tagi_conv2d_geom *g, const float *mu_w, const float *var_w, const float *mu_b,
                        const float *var_b, const float *mu_a, const float *var_a, int act, float *mu_a_out,
                        float *var_a_out, float *jcb_out, void *stream);
int tagi_conv2d_fwd_relu(const tagi_conv2d_geom *g, const float *mu_w, const float *var_w, const float *mu_b,
                         const float *var_b, const float *mu_a, const float *var_a, float *mu_a_out, float *var_a_out,
                         float *jcb_out, void *stream);

/* MixtureReLU moments (rectified Gaussian): alpha = mu_z / sqrt(var_z); mu_a = max(1e-6, mu_z * Phi(alpha) +
 * sqrt(var_z) * phi(alpha)); var_a = max(1e-6, -mu_a'^2 + 2 * mu_a' * mu_z - mu_z * sqrt(var_z) * phi(alpha) +
 * (var_z - mu_z^2) * Phi(alpha)) with mu_a' the unfloored mean; jcb = Phi(alpha).
 * CPU definition mixture_relu_mean_var (src/activation.cpp:152-178); replaces mixture_relu_mean_var_cuda
 * (src/activation_cuda.cu:130-157). */
int tagi_mixture_relu_fwd(const float *mu_z, const float *var_z, size_t n, float *mu_a, float *var_a, float *jcb,
                          void *stream);

/* Output-layer innovation, n entries: t = jcb / (var_a + var_obs); dmu = t * (obs - mu_a); dvar = -t * jcb; zero where t
 * is not finite or obs is NaN. CPU definition compute_delta_z_output (src/base_output_updater.cpp:8-29); replaces
 * update_delta_z_cuda (src/output_updater_cuda.cu:3-27). */
int tagi_output_delta(const float *mu_a, const float *var_a, const float *jcb, const float *obs, const float *var_obs,
                      size_t n, float *dmu, float *dvar, void *stream);

/* Index-selected innovation (hierarchical softmax): dmu / dvar (B * n_out entries) are zeroed, then for each of the
 * B * n_enc observations c the output unit selected_idx[c] (one-based within its sample) is updated as above.
 * CPU definition compute_selected_delta_z_output (src/base_output_updater.cpp:67-93, zeroing :281,300); replaces
 * update_delta_z_using_indices_cuda (src/output_updater_cuda.cu:29-60). selected_idx is a device array. */
int tagi_output_delta_selected(const float *mu_a, const float *var_a, const float *jcb, const float *obs,
                               const float *var_obs, const int *selected_idx, int B, int n_out, int n_enc, float *dmu,
                               float *dvar, void *stream);

/* Capped parameter update in place: mu += sign(dmu) * min(|dmu|, sqrt(var) / cap), var likewise, var <= 0 -> 1e-5;
 * cap = 0.1, 2, 3 for batch size 1, < 256, >= 256. neg_var_count (device int, may be NULL) is incremented per reset.
 * CPU definition BaseLayer::update_weights / update_biases (src/base_layer.cpp:116-187); replaces device_weight_update /
 * device_bias_update (src/base_layer_cuda.cu:56-103). */
int tagi_param_update(int batch_size, size_t n, float *mu, float *var, const float *dmu, const float *dvar,
                      int *neg_var_count, void *stream);

/* The same capped update for every parameter tensor of a network in one launch. `tensors` is a DEVICE array of n_tensors
 * descriptors (the caller builds it once; weights and biases of every layer are separate entries). The reference updates
 * layer by layer (Sequential::step -> update_weights / update_biases per layer, src/sequential.cpp:440-448) with a blocking
 * copy of the negative-variance counter after each; here the counter stays on the device. */
typedef struct {
    float *mu, *var;
    const float *dmu, *dvar;
    size_t n;
} tagi_param_tensor;
int tagi_param_update_multi(int batch_size, int n_tensors, const tagi_param_tensor *tensors, int *neg_var_count,
                            void *stream);

/* Same result as tagi_conv2d_bwd_param, for callers that must not allocate device memory while they run: a trainer
 * that gave the whole GPU to its own memory pool at start-up, a service with a fixed memory budget on a shared GPU, or
 * code running while another thread of the process captures a stream in the global capture mode (cudaMalloc is not
 * allowed then). This entry point has no counterpart in the reference. It never calls cudaMalloc, cudaFree or any
 * allocating routine: the partial sums of the split contraction go to a 16 MiB array that is part of the library
 * image (every GPU that loads the library holds it until the process exits).
 *  - Limit: fo * fi * k * k <= 1048576 weights (two slices of both partial tensors must fit); larger layers return
 *    TAGI_ERR_UNSUPPORTED with a message, use tagi_conv2d_bwd_param for them. Within the limit the contraction is cut
 *    into as many slices as fit, so results can differ from tagi_conv2d_bwd_param in the last bits.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device current);
 *    make that first call before any stream capture starts. With CUDA's lazy module loading the library's device code
 *    and the 16 MiB array are placed on a GPU by the first call of this library that launches on it, so make that call
 *    (this entry point, or any earlier Conv2d call) before the host's own pool takes the rest of the GPU's memory.
 *  - It always runs the FP32 FFMA kernels, so on layers the tensor-core path takes it is slower than
 *    tagi_conv2d_bwd_param (measured on a 64 -> 64 channel, 56 x 56, batch 64 layer: 2.2 ms against 0.74 ms).
 *  - All calls on a device share the array, which keeps whatever the previous call left; every call overwrites the part
 *    it reads, so nothing depends on old contents. Two calls that overlap on the GPU (different streams) race: keep
 *    calls of this entry point on one stream, or order them with events. */
int tagi_conv2d_bwd_param_noalloc(const tagi_conv2d_geom *g, const float *var_w, const float *var_b,
                                  const float *mu_a, const float *dmu_z, const float *dvar_z, float *dmu_w,
                                  float *dvar_w, float *dmu_b, float *dvar_b, void *stream);

/* ---- Layers between the Conv2d calls of the CNN / ResNet configurations: activations [B][C][H*W] ---- */

/* BatchNorm2d forward. training != 0: per-channel batch statistics mean = sum mu_a / n, var = (sum (mu_a - mean)^2 +
 * sum var_a) / (n - 1), n = B * wihi, written to mu_batch / var_batch; running averages updated in place as
 * ra = ra * momentum + batch * (1 - momentum) (the caller passes momentum 0 for the first training batch, as the
 * reference does); normalisation with the batch statistics. training == 0: normalisation with mu_ra / var_ra.
 * inv = 1 / sqrt(var + eps); mu_z = inv * (mu_a - mean) * mu_w + mu_b;
 * var_z = inv^2 * (var_a * (mu_w^2 + var_w) + var_w * (mu_a - mean)^2) + var_b.
 * CPU definition BatchNorm2d::forward (src/batchnorm_layer.cpp:15-26,127-206,849-985); replaces
 * batchnorm2d_stat_mean_var_cuda, batchnorm2d_sample_var_cuda, running_mean_var_cuda and batchnorm2d_fwd_mean_var_cuda
 * (src/batchnorm_layer_cuda.cu:141-152,439-543). */
int tagi_bn2d_fwd(int B, int C, int wihi, int has_bias, int training, float eps, float momentum, const float *mu_w,
                  const float *var_w, const float *mu_b, const float *var_b, const float *mu_a, const float *var_a,
                  float *mu_ra, float *var_ra, float *mu_batch, float *var_batch, float *mu_z, float *var_z,
                  void *stream);

/* BatchNorm2d backward in one pass. State deltas (state_update != 0): t = inv * mu_w * jcb; dmu = t * dmu_o;
 * dvar = t^2 * dvar_o (jcb NULL = 1). Parameter deltas per channel: dmu_w = sum u * dmu_o, dvar_w = sum u^2 * dvar_o with
 * u = inv * (mu_a - mean) * var_w; dmu_b = var_b * sum dmu_o, dvar_b = var_b^2 * sum dvar_o. mu_a / jcb are the layer's
 * saved input, mu_batch / var_batch the statistics of its forward pass.
 * CPU definition BatchNorm2d::backward (src/batchnorm_layer.cpp:233-255,307-357,987-1129, src/common.cpp:360-376);
 * replaces batchnorm2d_bwd_delta_z_cuda, batchnorm2d_bwd_delta_w_cuda, batchnorm2d_bwd_delta_b_cuda and
 * batchnorm2d_dual_sum_reduction (src/batchnorm_layer_cuda.cu:220-264,567-690). */
int tagi_bn2d_bwd(int B, int C, int wihi, int has_bias, int state_update, float eps, const float *mu_w,
                  const float *var_w, const float *var_b, const float *mu_a, const float *jcb, const float *mu_batch,
                  const float *var_batch, const float *dmu_o, const float *dvar_o, float *dmu, float *dvar, float *dmu_w,
                  float *dvar_w, float *dmu_b, float *dvar_b, void *stream);

/* AvgPool2d. The geometry is a tagi_conv2d_geom with fi = fo = channels (has_bias unused) and the same receptive-field
 * rule as Conv2d; taps in the padding contribute nothing while the divisors stay k*k (mean) and k^4 (variance).
 * Global pooling (kernel = image width, which pytagi writes as stride -1) is passed with stride = k.
 * Backward: dmu = jcb * (sum of dmu_o over the cells that contain the pixel) / k^2, dvar = jcb^2 * (...) / k^4.
 * CPU definition src/pooling_layer.cpp:59-176,207-375; replaces avgpool2d_fwd_(overlapped_)mean_var_cuda and
 * avgpool2d_bwd_(overlapped_)delta_z_cuda and their index tables (src/pooling_layer_cuda.cu:13-120). */
int tagi_avgpool2d_fwd(const tagi_conv2d_geom *g, const float *mu_a, const float *var_a, float *mu_z, float *var_z,
                       void *stream);
int tagi_avgpool2d_bwd_state(const tagi_conv2d_geom *g, const float *jcb, const float *dmu_o, const float *dvar_o,
                             float *dmu, float *dvar, void *stream);

/* Residual connection, in place on mu_a / var_a: mu_a += mu_s * j, var_a += var_s * j^2 (jcb NULL: j = 1).
 * CPU definition add_shortcut_mean_var / add_shortcut_delta (src/resnet_block.cpp:8-31); replaces
 * add_shortcut_mean_var_cuda / add_shortcut_delta_cuda (src/resnet_block_cuda.cu:7-33). */
int tagi_add_shortcut(const float *mu_s, const float *var_s, const float *jcb, size_t n, float *mu_a, float *var_a,
                      void *stream);

/* ---- Host I/O path of a training step ------------------------------------------------------------------------------
 * A pipeline owns `depth` slots. A slot holds, in pinned host memory and mirrored on the device, one batch's inputs
 * (in_floats), observations (obs_floats) and selected indices (idx_ints), and a pinned buffer for 2 * out_floats output
 * moments. The data loader writes a batch into the host buffers of a free slot; tagi_io_upload copies the slot to the
 * device asynchronously on the pipeline's own stream and makes compute_stream wait for it (a stream wait: the host does
 * not block), so the upload of batch i+1 overlaps the kernels of batch i. After the step's last kernel that reads the
 * slot's device buffers, tagi_io_consumed tells the pipeline the slot may be refilled. tagi_io_download copies exactly
 * n = B * n_out floats of mu and of var to the slot's pinned output buffer on a second stream after the work queued on
 * compute_stream so far, and tagi_io_wait_output blocks the host until they have landed.
 * Replaces, for the caller that adopts it, the blocking whole-buffer copies of cuTAGI's state carriers
 * (HiddenStateCuda::to_device / to_host, src/data_struct_cuda.cu:83-123: capacity = batch x widest layer, pageable host
 * vectors), ObservationCuda::to_device (src/data_struct_cuda.cu:300-330) and the list conversions of
 * pytagi/nn/output_updater.py:45-47. All allocations happen in tagi_io_create; no other call allocates.
 * One pipeline belongs to one device (the one current at creation) and one host thread. */
typedef struct tagi_io tagi_io;
int tagi_io_create(size_t in_floats, size_t obs_floats, size_t idx_ints, size_t out_floats, int depth, tagi_io **io);
int tagi_io_destroy(tagi_io *io);
/* Host (pinned) and device addresses of a slot's three input arrays; any of the out-pointers may be NULL. */
int tagi_io_host_buffers(tagi_io *io, int slot, float **inputs, float **obs, int **idx);
int tagi_io_device_buffers(tagi_io *io, int slot, const float **inputs, const float **obs, const int **idx);
int tagi_io_upload(tagi_io *io, int slot, void *compute_stream);
int tagi_io_consumed(tagi_io *io, int slot, void *compute_stream);
int tagi_io_download(tagi_io *io, int slot, const float *mu, const float *var, size_t n, void *compute_stream);
int tagi_io_wait_output(tagi_io *io, int slot, const float **mu, const float **var);

#ifdef __cplusplus
}
#endif
#endif /* TAGI_B200_H */
