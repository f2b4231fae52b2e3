// Shared host-side helpers of the C-ABI translation units: status codes, the per-thread error
// string and argument checks.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <initializer_list>
#include <string>

#include "../../include/tagi_b200.h"

namespace tagi {

std::string &last_error();  // thread-local
int fail(int code, const std::string &msg);
int cuda_fail(cudaError_t e, const char *where);

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned4(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 3u) == 0; }

#define TAGI_REQUIRE(cond, msg) \
    do {                        \
        if (!(cond)) return ::tagi::fail(TAGI_ERR_INVALID_ARGUMENT, std::string(__func__) + ": " + (msg)); \
    } while (0)

#define TAGI_CUDA(expr)                                                  \
    do {                                                                 \
        cudaError_t e__ = (expr);                                        \
        if (e__ != cudaSuccess) return ::tagi::cuda_fail(e__, #expr);    \
    } while (0)

int current_impl();  // TAGI_IMPL_*

// FFMA implementations (tagi_linear_ffma.cu)
int linear_fwd_ffma(const float *mu_w, const float *var_w, const float *mu_b, const float *var_b, const float *mu_a,
                    const float *var_a, int B, int K, int N, float *mu_z, float *var_z, cudaStream_t st);
int linear_bwd_state_ffma(const float *mu_w, const float *jcb, const float *dmu_z, const float *dvar_z, int B, int K,
                          int N, float *dmu_a, float *dvar_a, cudaStream_t st);
int linear_bwd_param_ffma(const float *var_w, const float *mu_a, const float *dmu_z, const float *dvar_z, int B,
                          int K, int N, float *dmu_w, float *dvar_w, cudaStream_t st, long ldz = 0);
// column sums of the [B][N] deltas scaled by var_b, var_b^2
int linear_bias_delta(const float *var_b, const float *dmu_z, const float *dvar_z, int B, int N, float *dmu_b,
                      float *dvar_b, cudaStream_t st, long ldz = 0);

// tcgen05 / 3xTF32 implementations (tagi_linear_tc.cu)
bool linear_tc_supported(int B, int K, int N, std::initializer_list<const void *> ptrs);
bool linear_tc_profitable(int B, int K, int N);
int linear_tc_set_chunked(int on);
int linear_tc_set_sm_budget(int sms);
int linear_tc_set_variant(int v);
int linear_tc_status(int *out, int reset);
// Implicit Conv2d operand for the pair kernel's A side (forward: receptive fields of the activations; state pass at
// stride 1: the deltas each input pixel receives). Row R of A is pixel (b, py, px) of a pixel grid OHW / OW per image,
// column kc = (c, ky, kx); its value is src[b][c][y0 + sign * ky][x0 + sign * kx] with
//   sign = +1: y0 = py * stride - off,  x0 = px * stride - off      (im2col)
//   sign = -1: y0 = py + off,           x0 = px + off               (delta gather)
// and zero outside the source image. on == 0: A tiles come by TMA from a matrix in memory.
struct ConvGather {
    int on;
    const float *s0, *s1;
    int C, H, W, OW, OHW, k, stride, off, sign;
    long rows;
};

int linear_fwd_tc(const float *mu_w, const float *var_w, const float *mu_b, const float *var_b, const float *mu_a,
                  const float *var_a, int B, int K, int N, float *mu_z, float *var_z, cudaStream_t st, int npix = 0,
                  const ConvGather *cg = nullptr, float *relu_jcb = nullptr);
// relu_jcb (only when linear_tc_pair_for(B)): the ReLU is folded into the epilogue; mu_z / var_z receive the moments
// after the ReLU and relu_jcb its Jacobian
bool linear_tc_pair_for(int rows);  // true when a pass with this many output rows runs on the CTA-pair kernel
int linear_bwd_state_tc(const float *mu_w, const float *jcb, const float *dmu_z, const float *dvar_z, int B, int K,
                        int N, float *dmu_a, float *dvar_a, cudaStream_t st, int npix = 0,
                        const ConvGather *cg = nullptr);
// npix > 0: the rows are (image, pixel) pairs and outputs / the Jacobian are laid out [image][channel][pixel] (Conv2d)
int linear_bwd_param_tc(const float *var_w, const float *mu_a, const float *dmu_z, const float *dvar_z, int B, int K,
                        int N, float *dmu_w, float *dvar_w, cudaStream_t st, float *split_ws = nullptr, int slices = 1,
                        long ldz = 0, const float *var_b = nullptr, float *dmu_b = nullptr, float *dvar_b = nullptr);
// true: the parameter pass of N output features (without a split contraction) can produce the bias deltas itself when it
// is given var_b / dmu_b / dvar_b, so that linear_bias_delta's pass over the deltas is not needed
bool linear_bwd_param_tc_fuses_bias(int N);
int linear_bwd_param_tc_slices(int B, int K, int N);

// Conv2d on the FFMA engine (tagi_conv_ffma.cu)
int conv2d_fwd_ffma(const tagi_conv2d_geom &g, const float *mu_w, const float *var_w, const float *mu_b,
                    const float *var_b, const float *mu_a, const float *var_a, float *mu_z, float *var_z,
                    cudaStream_t st);
int conv2d_bwd_state_ffma(const tagi_conv2d_geom &g, const float *mu_w, const float *jcb, const float *dmu_z,
                          const float *dvar_z, float *dmu_a, float *dvar_a, cudaStream_t st);
int conv2d_bwd_param_ffma(const tagi_conv2d_geom &g, const float *var_w, const float *var_b, const float *mu_a,
                          const float *dmu_z, const float *dvar_z, float *dmu_w, float *dvar_w, float *dmu_b,
                          float *dvar_b, cudaStream_t st);
// Library-owned scratch of the current device, grow-only; st = the stream the caller launches on (growth is refused
// while that stream is being captured). Blocks that were handed out are retired, not freed, when a larger one is needed.
int conv_scratch(size_t bytes, float **out, cudaStream_t st);
int reserve_scratch(size_t bytes);
size_t conv_tc_workspace_bytes(const tagi_conv2d_geom &g);
size_t conv_ffma_workspace_bytes(const tagi_conv2d_geom &g);
int release_scratch();
size_t scratch_bytes();
int conv_bias_delta(const tagi_conv2d_geom &g, const float *var_b, const float *dmu_z, const float *dvar_z,
                    float *dmu_b, float *dvar_b, cudaStream_t st);
// Conv2d on the tensor-core Linear kernels (tagi_conv_tc.cu)
enum { CONV_PASS_FWD = 0, CONV_PASS_STATE = 1, CONV_PASS_PARAM = 2 };
bool conv_tc_supported(const tagi_conv2d_geom &g, int pass, std::initializer_list<const void *> ptrs);
bool conv_tc_profitable(const tagi_conv2d_geom &g, int pass);
int conv2d_fwd_tc(const tagi_conv2d_geom &g, const float *mu_w, const float *var_w, const float *mu_b,
                  const float *var_b, const float *mu_a, const float *var_a, float *mu_z, float *var_z,
                  cudaStream_t st, float *relu_jcb = nullptr);
bool conv2d_fwd_tc_fuses_relu(const tagi_conv2d_geom &g);  // the forward of this geometry runs on the CTA-pair kernel
int conv2d_bwd_state_tc(const tagi_conv2d_geom &g, const float *mu_w, const float *jcb, const float *dmu_z,
                        const float *dvar_z, float *dmu_a, float *dvar_a, cudaStream_t st);
int conv2d_bwd_param_tc(const tagi_conv2d_geom &g, const float *var_w, const float *mu_a, const float *dmu_z,
                        const float *dvar_z, float *dmu_w, float *dvar_w, cudaStream_t st);
// Implicit-GEMM parameter pass on the tensor cores (tagi_conv_patch.cu): operands read by TMA as they lie in memory
bool conv_param_patch_supported(const tagi_conv2d_geom &g, std::initializer_list<const void *> ptrs);
size_t conv_param_patch_workspace_bytes(const tagi_conv2d_geom &g);
int conv2d_bwd_param_patch(const tagi_conv2d_geom &g, const float *var_w, const float *mu_a, const float *dmu_z,
                           const float *dvar_z, float *dmu_w, float *dvar_w, cudaStream_t st);
// Implicit-GEMM forward and stride-1 state pass with TMA-loaded patches (tagi_conv_patch.cu)
bool conv_pix_patch_supported(const tagi_conv2d_geom &g, int pass, std::initializer_list<const void *> ptrs);
size_t conv_pix_patch_workspace_bytes(const tagi_conv2d_geom &g);
int conv2d_fwd_patch(const tagi_conv2d_geom &g, const float *mu_w, const float *var_w, const float *mu_b, const float *var_b,
                     const float *mu_a, const float *var_a, float *mu_z, float *var_z, cudaStream_t st, float *relu_jcb);
int conv2d_bwd_state_patch(const tagi_conv2d_geom &g, const float *mu_w, const float *jcb, const float *dmu_z,
                           const float *dvar_z, float *dmu_a, float *dvar_a, cudaStream_t st);
int conv2d_bwd_param_noalloc(const tagi_conv2d_geom &g, const float *var_w, const float *var_b, const float *mu_a,
                             const float *dmu_z, const float *dvar_z, float *dmu_w, float *dvar_w, float *dmu_b,
                             float *dvar_b, cudaStream_t st);

}  // namespace tagi
