// TAGI Linear on the FP32 FFMA tile engine: forward, state-delta backward, parameter-delta backward.
// Arithmetic follows the reference's CPU definitions (src/linear_layer.cpp:10-60, 245-272, 314-349,
// 391-423 of cuTAGI); the reference's own CUDA launchers for the same three steps are
// src/linear_layer_cuda.cu:12-168.
#include "tagi_common.h"
#include "tagi_ffma.cuh"

namespace tagi {
namespace {

inline int done(cudaError_t e) { return e == cudaSuccess ? TAGI_OK : cuda_fail(e, "FFMA tile kernel launch"); }

// Column sums of the deltas: one CTA per 32 columns, 8 row lanes, fixed-order reduction so the
// result does not depend on scheduling.
__global__ void __launch_bounds__(256) bias_delta_kernel(const float *__restrict__ var_b,
                                                         const float *__restrict__ dmu_z,
                                                         const float *__restrict__ dvar_z, int B, int N, long ld,
                                                         float *__restrict__ dmu_b, float *__restrict__ dvar_b) {
    __shared__ float s1[8][33], s2[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int n = blockIdx.x * 32 + tx;
    float a1 = 0.f, a2 = 0.f;
    if (n < N)
        for (int b = ty; b < B; b += 8) {
            a1 += __ldg(dmu_z + (long)b * ld + n);
            a2 += __ldg(dvar_z + (long)b * ld + n);
        }
    s1[ty][tx] = a1;
    s2[ty][tx] = a2;
    __syncthreads();
    if (ty == 0 && n < N) {
#pragma unroll
        for (int i = 1; i < 8; i++) {
            a1 += s1[i][tx];
            a2 += s2[i][tx];
        }
        const float vb = __ldg(var_b + n);
        dmu_b[n] = a1 * vb;
        dvar_b[n] = a2 * vb * vb;
    }
}

}  // namespace

int linear_fwd_ffma(const float *mu_w, const float *var_w, const float *mu_b, const float *var_b, const float *mu_a,
                    const float *var_a, int B, int K, int N, float *mu_z, float *var_z, cudaStream_t st) {
    StridedOperand<DER_MEAN_VAR_ACT> A{mu_a, var_a, (long)K, 1, B, K};
    StridedOperand<DER_MEAN_VAR_W> W{mu_w, var_w, (long)K, 1, N, K};
    EpiRowBias epi{mu_z, var_z, mu_b, var_b, (long)N,
                   N % 4 == 0 && aligned16(mu_z) && aligned16(var_z) &&
                       (!mu_b || (aligned16(mu_b) && aligned16(var_b)))};
    const bool kv = K % 4 == 0;
    return done(dispatch_ffma<decltype(A), decltype(W), EpiRowBias, LOAD_K_VEC4, LOAD_K_SCALAR, LOAD_K_VEC4, LOAD_K_SCALAR>(
        A, W, epi, B, N, K, kv && aligned16(mu_a) && aligned16(var_a), kv && aligned16(mu_w) && aligned16(var_w), st));
}

int linear_bwd_state_ffma(const float *mu_w, const float *jcb, const float *dmu_z, const float *dvar_z, int B, int K,
                          int N, float *dmu_a, float *dvar_a, cudaStream_t st) {
    // rows = batch, columns = input features, contraction over the output features
    StridedOperand<DER_PAIR> A{dmu_z, dvar_z, (long)N, 1, B, N};
    StridedOperand<DER_SQUARE> W{mu_w, nullptr, 1, (long)K, K, N};
    EpiRowScale epi{dmu_a, dvar_a, jcb, (long)K,
                    K % 4 == 0 && aligned16(dmu_a) && aligned16(dvar_a) && (!jcb || aligned16(jcb))};
    return done(dispatch_ffma<decltype(A), decltype(W), EpiRowScale, LOAD_K_VEC4, LOAD_K_SCALAR, LOAD_R_VEC4, LOAD_R_SCALAR>(
        A, W, epi, B, K, N, N % 4 == 0 && aligned16(dmu_z) && aligned16(dvar_z), K % 4 == 0 && aligned16(mu_w), st));
}

int linear_bwd_param_ffma(const float *var_w, const float *mu_a, const float *dmu_z, const float *dvar_z, int B,
                          int K, int N, float *dmu_w, float *dvar_w, cudaStream_t st, long ldz) {
    // rows = output features, columns = input features, contraction over the batch; ldz: row pitch of the delta
    // matrices (more than N when only a range of the output features is computed)
    if (ldz == 0) ldz = N;
    StridedOperand<DER_PAIR> A{dmu_z, dvar_z, 1, ldz, N, B};
    StridedOperand<DER_SQUARE> X{mu_a, nullptr, 1, (long)K, K, B};
    EpiRowScale epi{dmu_w, dvar_w, var_w, (long)K,
                    K % 4 == 0 && aligned16(dmu_w) && aligned16(dvar_w) && aligned16(var_w)};
    return done(dispatch_ffma<decltype(A), decltype(X), EpiRowScale, LOAD_R_VEC4, LOAD_R_SCALAR, LOAD_R_VEC4, LOAD_R_SCALAR>(
        A, X, epi, N, K, B, N % 4 == 0 && aligned16(dmu_z) && aligned16(dvar_z), K % 4 == 0 && aligned16(mu_a), st));
}

int linear_bias_delta(const float *var_b, const float *dmu_z, const float *dvar_z, int B, int N, float *dmu_b,
                      float *dvar_b, cudaStream_t st, long ldz) {
    bias_delta_kernel<<<(N + 31) / 32, 256, 0, st>>>(var_b, dmu_z, dvar_z, B, N, ldz ? ldz : N, dmu_b, dvar_b);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "bias_delta_kernel launch");
    return TAGI_OK;
}

}  // namespace tagi
