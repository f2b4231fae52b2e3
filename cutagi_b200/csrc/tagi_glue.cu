// Elementwise neighbours of the hot path, so that whole TAGI training steps can run on the device through this
// library alone: ReLU moments, output-layer innovation (plain and index-selected), capped parameter update.
// Each follows the reference's CPU definition; the reference's CUDA counterparts are cited at the entry points.
#include "tagi_common.h"

namespace tagi {
namespace {

constexpr int BLOCK = 256;
inline unsigned blocks_for(size_t n) { return (unsigned)((n + BLOCK - 1) / BLOCK); }

// src/activation.cpp:7-29
__device__ __forceinline__ void relu_one(float mz, float vz, float &ma, float &va, float &j) {
    ma = fmaxf(mz, 0.f);
    if (ma == 0.f) {
        j = 0.f;
        va = 0.f;
    } else {
        j = 1.f;
        va = vz;
    }
}
// The activation kernels may run in place (mu_a == mu_z, var_a == var_z): no __restrict__, no read-only loads; every
// thread reads its own elements before it writes them.
__global__ void relu_kernel(const float *mu_z, const float *var_z, size_t n, float *mu_a, float *var_a, float *jcb) {
    const size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x;
    if (i >= n) return;
    relu_one(mu_z[i], var_z[i], mu_a[i], var_a[i], jcb[i]);
}
// four elements per thread with 16-byte accesses (n a multiple of 4, 16-byte aligned tensors)
__global__ void relu_vec4_kernel(const float4 *mu_z, const float4 *var_z, size_t n4, float4 *mu_a, float4 *var_a,
                                 float4 *jcb) {
    const size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x;
    if (i >= n4) return;
    const float4 m = mu_z[i], v = var_z[i];
    float4 a, va, j;
    relu_one(m.x, v.x, a.x, va.x, j.x);
    relu_one(m.y, v.y, a.y, va.y, j.y);
    relu_one(m.z, v.z, a.z, va.z, j.z);
    relu_one(m.w, v.w, a.w, va.w, j.w);
    mu_a[i] = a;
    var_a[i] = va;
    jcb[i] = j;
}

// src/activation.cpp:152-178 (rectified-Gaussian moments; Phi by erfc as in src/common.cpp:315-319)
__device__ __forceinline__ void mixture_relu_one(float m, float v, float &ma, float &va, float &j) {
    constexpr float SQRT_2PI = 2.5066282746310002f;
    const float sd = sqrtf(v), alpha = m / sd;
    const float pdf = (1.0f / SQRT_2PI) * expf(-0.5f * alpha * alpha);
    const float cdf = 0.5f * erfcf(-alpha * 0.7071067811865475f);
    const float t = m * cdf + sd * pdf;
    ma = fmaxf(0.000001f, t);
    va = fmaxf(0.000001f, -t * t + 2 * t * m - m * sd * pdf + (v - m * m) * cdf);
    j = cdf;
}
__global__ void mixture_relu_kernel(const float *mu_z, const float *var_z, size_t n, float *mu_a, float *var_a,
                                    float *jcb) {
    const size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x;
    if (i >= n) return;
    float ma, va, j;
    mixture_relu_one(mu_z[i], var_z[i], ma, va, j);
    mu_a[i] = ma;
    var_a[i] = va;
    jcb[i] = j;
}
// four elements per thread with 16-byte accesses (n a multiple of 4, 16-byte aligned tensors)
__global__ void mixture_relu_vec4_kernel(const float4 *mu_z, const float4 *var_z, size_t n4, float4 *mu_a, float4 *var_a,
                                         float4 *jcb) {
    const size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x;
    if (i >= n4) return;
    const float4 m = mu_z[i], v = var_z[i];
    float4 a, va, j;
    mixture_relu_one(m.x, v.x, a.x, va.x, j.x);
    mixture_relu_one(m.y, v.y, a.y, va.y, j.y);
    mixture_relu_one(m.z, v.z, a.z, va.z, j.z);
    mixture_relu_one(m.w, v.w, a.w, va.w, j.w);
    mu_a[i] = a;
    var_a[i] = va;
    jcb[i] = j;
}

// src/base_output_updater.cpp:8-29
__global__ void output_delta_kernel(const float *__restrict__ mu_a, const float *__restrict__ var_a,
                                    const float *__restrict__ jcb, const float *__restrict__ obs,
                                    const float *__restrict__ var_obs, size_t n, float *__restrict__ dmu,
                                    float *__restrict__ dvar) {
    const size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x;
    if (i >= n) return;
    const float t = jcb[i] / (var_a[i] + var_obs[i]);
    if (isinf(t) || isnan(t) || isnan(obs[i])) {
        dmu[i] = 0.f;
        dvar[i] = 0.f;
    } else {
        dmu[i] = t * (obs[i] - mu_a[i]);
        dvar[i] = -t * jcb[i];
    }
}

// src/base_output_updater.cpp:67-93; selected_idx is one-based within a sample
__global__ void output_delta_selected_kernel(const float *__restrict__ mu_a, const float *__restrict__ var_a,
                                             const float *__restrict__ jcb, const float *__restrict__ obs,
                                             const float *__restrict__ var_obs, const int *__restrict__ sel, int n_sel,
                                             int n_out, int n_enc, float *__restrict__ dmu,
                                             float *__restrict__ dvar) {
    const int c = blockIdx.x * BLOCK + threadIdx.x;
    if (c >= n_sel) return;
    const long idx = sel[c] + (long)(c / n_enc) * n_out - 1;
    const float t = jcb[idx] / (var_a[idx] + var_obs[c]);
    if (isinf(t) || isnan(t)) {
        dmu[idx] = 0.f;
        dvar[idx] = 0.f;
    } else {
        dmu[idx] = t * (obs[c] - mu_a[idx]);
        dvar[idx] = -t * jcb[idx];
    }
}

// src/base_layer.cpp:116-162
__global__ void param_update_kernel(const float *__restrict__ dmu, const float *__restrict__ dvar, float cap, size_t n,
                                    float *__restrict__ mu, float *__restrict__ var, int *__restrict__ neg) {
    const size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x;
    if (i >= n) return;
    const float dm = dmu[i], dv = dvar[i];
    const float sm = (float)((dm > 0.f) - (dm < 0.f)), sv = (float)((dv > 0.f) - (dv < 0.f));
    float v = var[i];
    const float bar = sqrtf(v) / cap;
    mu[i] += sm * fminf(fabsf(dm), bar);
    v += sv * fminf(fabsf(dv), bar);
    if (v <= 0.f) {
        v = 1e-5f;
        if (neg) atomicAdd(neg, 1);
    }
    var[i] = v;
}

inline int launched(const char *what) {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? TAGI_OK : cuda_fail(e, what);
}

// The same update for a table of tensors (device array), one launch: blockIdx.y selects the tensor
__global__ void param_update_multi_kernel(const tagi_param_tensor *__restrict__ t, float cap, int *__restrict__ neg) {
    const tagi_param_tensor x = t[blockIdx.y];
    for (size_t i = (size_t)blockIdx.x * BLOCK + threadIdx.x; i < x.n; i += (size_t)gridDim.x * BLOCK) {
        const float dm = x.dmu[i], dv = x.dvar[i];
        const float sm = (float)((dm > 0.f) - (dm < 0.f)), sv = (float)((dv > 0.f) - (dv < 0.f));
        float v = x.var[i];
        const float bar = sqrtf(v) / cap;
        x.mu[i] += sm * fminf(fabsf(dm), bar);
        v += sv * fminf(fabsf(dv), bar);
        if (v <= 0.f) {
            v = 1e-5f;
            if (neg) atomicAdd(neg, 1);
        }
        x.var[i] = v;
    }
}

}  // namespace
}  // namespace tagi

using namespace tagi;

#define TAGI_PTR(p) TAGI_REQUIRE((p) != nullptr && aligned4(p), #p " is null or not 4-byte aligned")

extern "C" {

int tagi_relu_fwd(const float *mu_z, const float *var_z, size_t n, float *mu_a, float *var_a, float *jcb,
                  void *stream) {
    TAGI_REQUIRE(n > 0, "n must be positive");
    TAGI_PTR(mu_z);
    TAGI_PTR(var_z);
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    TAGI_PTR(jcb);
    if (n % 4 == 0 && aligned16(mu_z) && aligned16(var_z) && aligned16(mu_a) && aligned16(var_a) && aligned16(jcb))
        relu_vec4_kernel<<<blocks_for(n / 4), BLOCK, 0, static_cast<cudaStream_t>(stream)>>>(
            reinterpret_cast<const float4 *>(mu_z), reinterpret_cast<const float4 *>(var_z), n / 4,
            reinterpret_cast<float4 *>(mu_a), reinterpret_cast<float4 *>(var_a), reinterpret_cast<float4 *>(jcb));
    else
        relu_kernel<<<blocks_for(n), BLOCK, 0, static_cast<cudaStream_t>(stream)>>>(mu_z, var_z, n, mu_a, var_a, jcb);
    return launched("relu_kernel launch");
}

int tagi_mixture_relu_fwd(const float *mu_z, const float *var_z, size_t n, float *mu_a, float *var_a, float *jcb,
                          void *stream) {
    TAGI_REQUIRE(n > 0, "n must be positive");
    TAGI_PTR(mu_z);
    TAGI_PTR(var_z);
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    TAGI_PTR(jcb);
    if (n % 4 == 0 && aligned16(mu_z) && aligned16(var_z) && aligned16(mu_a) && aligned16(var_a) && aligned16(jcb))
        mixture_relu_vec4_kernel<<<blocks_for(n / 4), BLOCK, 0, static_cast<cudaStream_t>(stream)>>>(
            reinterpret_cast<const float4 *>(mu_z), reinterpret_cast<const float4 *>(var_z), n / 4,
            reinterpret_cast<float4 *>(mu_a), reinterpret_cast<float4 *>(var_a), reinterpret_cast<float4 *>(jcb));
    else
        mixture_relu_kernel<<<blocks_for(n), BLOCK, 0, static_cast<cudaStream_t>(stream)>>>(mu_z, var_z, n, mu_a, var_a,
                                                                                             jcb);
    return launched("mixture_relu_kernel launch");
}

int tagi_output_delta(const float *mu_a, const float *var_a, const float *jcb, const float *obs, const float *var_obs,
                      size_t n, float *dmu, float *dvar, void *stream) {
    TAGI_REQUIRE(n > 0, "n must be positive");
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    TAGI_PTR(jcb);
    TAGI_PTR(obs);
    TAGI_PTR(var_obs);
    TAGI_PTR(dmu);
    TAGI_PTR(dvar);
    output_delta_kernel<<<blocks_for(n), BLOCK, 0, static_cast<cudaStream_t>(stream)>>>(mu_a, var_a, jcb, obs, var_obs,
                                                                                         n, dmu, dvar);
    return launched("output_delta_kernel launch");
}

int tagi_output_delta_selected(const float *mu_a, const float *var_a, const float *jcb, const float *obs,
                               const float *var_obs, const int *selected_idx, int B, int n_out, int n_enc, float *dmu,
                               float *dvar, void *stream) {
    TAGI_REQUIRE(B > 0 && n_out > 0 && n_enc > 0, "B, n_out and n_enc must be positive");
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    TAGI_PTR(jcb);
    TAGI_PTR(obs);
    TAGI_PTR(var_obs);
    TAGI_PTR(selected_idx);
    TAGI_PTR(dmu);
    TAGI_PTR(dvar);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t bytes = (size_t)B * n_out * sizeof(float);
    TAGI_CUDA(cudaMemsetAsync(dmu, 0, bytes, st));
    TAGI_CUDA(cudaMemsetAsync(dvar, 0, bytes, st));
    const int n_sel = B * n_enc;
    output_delta_selected_kernel<<<blocks_for(n_sel), BLOCK, 0, st>>>(mu_a, var_a, jcb, obs, var_obs, selected_idx,
                                                                      n_sel, n_out, n_enc, dmu, dvar);
    return launched("output_delta_selected_kernel launch");
}

int tagi_param_update_multi(int batch_size, int n_tensors, const tagi_param_tensor *tensors, int *neg_var_count,
                            void *stream) {
    TAGI_REQUIRE(batch_size > 0 && n_tensors > 0, "batch_size and n_tensors must be positive");
    TAGI_REQUIRE(tensors != nullptr, "tensors is null");
    const float cap = batch_size == 1 ? 0.1f : (batch_size < 256 ? 2.0f : 3.0f);
    // one CTA column per tensor, 148 * 4 CTAs along each tensor (grid-stride): one launch for the whole network
    param_update_multi_kernel<<<dim3(148 * 4, n_tensors), BLOCK, 0, static_cast<cudaStream_t>(stream)>>>(tensors, cap,
                                                                                                       neg_var_count);
    return launched("param_update_multi_kernel launch");
}

int tagi_param_update(int batch_size, size_t n, float *mu, float *var, const float *dmu, const float *dvar,
                      int *neg_var_count, void *stream) {
    TAGI_REQUIRE(batch_size > 0 && n > 0, "batch_size and n must be positive");
    TAGI_PTR(mu);
    TAGI_PTR(var);
    TAGI_PTR(dmu);
    TAGI_PTR(dvar);
    // cap factor: 0.1 for batch 1, 2 below 256, 3 from 256 on (src/base_layer.cpp:164-187)
    const float cap = batch_size == 1 ? 0.1f : (batch_size < 256 ? 2.0f : 3.0f);
    param_update_kernel<<<blocks_for(n), BLOCK, 0, static_cast<cudaStream_t>(stream)>>>(dmu, dvar, cap, n, mu, var,
                                                                                        neg_var_count);
    return launched("param_update_kernel launch");
}

}  // extern "C"
