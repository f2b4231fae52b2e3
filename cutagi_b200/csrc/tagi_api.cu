// C-ABI entry points (include/tagi_b200.h): argument checks, implementation choice, status codes.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "tagi_common.h"

namespace tagi {

std::string &last_error() {
    static thread_local std::string s;
    return s;
}
int fail(int code, const std::string &msg) {
    last_error() = msg;
    return code;
}
int cuda_fail(cudaError_t e, const char *where) {
    last_error() = std::string(where) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
    return TAGI_ERR_CUDA;
}

namespace {
std::atomic<int> g_impl{-1};
int impl_from_env() {
    const char *v = std::getenv("TAGI_B200_IMPL");
    if (!v) return TAGI_IMPL_AUTO;
    if (!std::strcmp(v, "ffma")) return TAGI_IMPL_FFMA;
    if (!std::strcmp(v, "tf32x3")) return TAGI_IMPL_TF32X3;
    return TAGI_IMPL_AUTO;
}
}  // namespace
int current_impl() {
    int impl = g_impl;
    if (impl < 0) {
        impl = impl_from_env();
        g_impl = impl;
    }
    return impl;
}

}  // namespace tagi

using namespace tagi;

extern "C" {

const char *tagi_last_error_string(void) { return last_error().c_str(); }
int tagi_version(void) { return 100; }

int tagi_set_impl(int impl) {
    TAGI_REQUIRE(impl >= TAGI_IMPL_AUTO && impl <= TAGI_IMPL_TF32X3, "unknown implementation id");
    g_impl = impl;
    return TAGI_OK;
}
int tagi_get_impl(void) { return current_impl(); }

int tagi_tc_status(int *status, int reset) {
    TAGI_REQUIRE(status != nullptr, "null status pointer");
    return linear_tc_status(status, reset);
}
int tagi_reserve_scratch(size_t bytes) { return reserve_scratch(bytes); }
int tagi_release_scratch(void) { return release_scratch(); }
size_t tagi_scratch_bytes(void) { return scratch_bytes(); }
int tagi_tc_set_chunked(int on) { return linear_tc_set_chunked(on); }
int tagi_tc_set_sm_budget(int sms) { return linear_tc_set_sm_budget(sms); }
int tagi_tc_set_variant(int v) { return linear_tc_set_variant(v); }

// true -> run the tensor-core kernel; sets rc when the forced implementation cannot take the shape
static bool pick_tc(const char *who, int B, int K, int N, std::initializer_list<const void *> ptrs, int *rc) {
    *rc = TAGI_OK;
    const int impl = current_impl();
    if (impl == TAGI_IMPL_FFMA) return false;
    const bool ok = linear_tc_supported(B, K, N, ptrs);
    if (impl == TAGI_IMPL_TF32X3) {
        if (!ok)
            *rc = fail(TAGI_ERR_UNSUPPORTED, std::string(who) + ": TF32X3 needs 16-byte aligned tensors and B, K, N "
                                                               "that are multiples of 4");
        return ok;
    }
    return ok && linear_tc_profitable(B, K, N);
}

#define TAGI_PTR(p) TAGI_REQUIRE((p) != nullptr && aligned4(p), #p " is null or not 4-byte aligned")
#define TAGI_DIMS()                                                                            \
    TAGI_REQUIRE(B > 0 && K > 0 && N > 0, "B, K and N must be positive");                        \
    TAGI_REQUIRE((long)B * K < (1L << 31) && (long)B * N < (1L << 31) && (long)K * N < (1L << 31), \
                 "tensor extent exceeds 2^31 elements")

int tagi_linear_fwd(const float *mu_w, const float *var_w, const float *mu_b, const float *var_b, const float *mu_a,
                    const float *var_a, int B, int K, int N, int has_bias, float *mu_z, float *var_z, void *stream) {
    TAGI_DIMS();
    TAGI_PTR(mu_w);
    TAGI_PTR(var_w);
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    TAGI_PTR(mu_z);
    TAGI_PTR(var_z);
    if (has_bias) {
        TAGI_PTR(mu_b);
        TAGI_PTR(var_b);
    } else {
        mu_b = var_b = nullptr;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    if (pick_tc(__func__, B, K, N, {mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_z, var_z}, &rc))
        return linear_fwd_tc(mu_w, var_w, mu_b, var_b, mu_a, var_a, B, K, N, mu_z, var_z, st);
    if (rc != TAGI_OK) return rc;
    return linear_fwd_ffma(mu_w, var_w, mu_b, var_b, mu_a, var_a, B, K, N, mu_z, var_z, st);
}

static int act_after(int act, float *mu, float *var, size_t n, float *jcb, void *stream) {
    return act == TAGI_ACT_RELU ? tagi_relu_fwd(mu, var, n, mu, var, jcb, stream)
                                : tagi_mixture_relu_fwd(mu, var, n, mu, var, jcb, stream);
}

int tagi_linear_fwd_act(const float *mu_w, const float *var_w, const float *mu_b, const float *var_b, const float *mu_a,
                        const float *var_a, int B, int K, int N, int has_bias, int act, float *mu_a_out, float *var_a_out,
                        float *jcb_out, void *stream) {
    TAGI_DIMS();
    TAGI_REQUIRE(act == TAGI_ACT_RELU || act == TAGI_ACT_MIXTURE_RELU, "unknown activation id");
    TAGI_PTR(mu_w);
    TAGI_PTR(var_w);
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    TAGI_PTR(mu_a_out);
    TAGI_PTR(var_a_out);
    TAGI_PTR(jcb_out);
    if (has_bias) {
        TAGI_PTR(mu_b);
        TAGI_PTR(var_b);
    } else {
        mu_b = var_b = nullptr;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    // ReLU: one kernel where the forward runs on CTA pairs. Otherwise, and for the MixtureReLU (whose erf / exp arithmetic
    // in the epilogue, 64 columns per thread, was measured slower than a pass of its own), the forward followed by the
    // activation in place.
    if (pick_tc(__func__, B, K, N, {mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_a_out, var_a_out, jcb_out}, &rc) &&
        linear_tc_pair_for(B) && act == TAGI_ACT_RELU)
        return linear_fwd_tc(mu_w, var_w, mu_b, var_b, mu_a, var_a, B, K, N, mu_a_out, var_a_out, st, 0, nullptr, jcb_out);
    if (rc != TAGI_OK) return rc;
    rc = tagi_linear_fwd(mu_w, var_w, mu_b, var_b, mu_a, var_a, B, K, N, has_bias, mu_a_out, var_a_out, stream);
    if (rc != TAGI_OK) return rc;
    return act_after(act, mu_a_out, var_a_out, (size_t)B * N, jcb_out, stream);
}

int tagi_linear_fwd_relu(const float *mu_w, const float *var_w, const float *mu_b, const float *var_b, const float *mu_a,
                         const float *var_a, int B, int K, int N, int has_bias, float *mu_a_out, float *var_a_out,
                         float *jcb_out, void *stream) {
    return tagi_linear_fwd_act(mu_w, var_w, mu_b, var_b, mu_a, var_a, B, K, N, has_bias, TAGI_ACT_RELU, mu_a_out, var_a_out,
                               jcb_out, stream);
}

int tagi_linear_bwd_state(const float *mu_w, const float *jcb, const float *dmu_z, const float *dvar_z, int B, int K,
                          int N, float *dmu_a, float *dvar_a, void *stream) {
    TAGI_DIMS();
    TAGI_PTR(mu_w);
    if (jcb) TAGI_PTR(jcb);
    TAGI_PTR(dmu_z);
    TAGI_PTR(dvar_z);
    TAGI_PTR(dmu_a);
    TAGI_PTR(dvar_a);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    if (pick_tc(__func__, B, K, N, {mu_w, jcb, dmu_z, dvar_z, dmu_a, dvar_a}, &rc))
        return linear_bwd_state_tc(mu_w, jcb, dmu_z, dvar_z, B, K, N, dmu_a, dvar_a, st);
    if (rc != TAGI_OK) return rc;
    return linear_bwd_state_ffma(mu_w, jcb, dmu_z, dvar_z, B, K, N, dmu_a, dvar_a, st);
}

int tagi_linear_bwd_param(const float *var_w, const float *var_b, const float *mu_a, const float *dmu_z,
                          const float *dvar_z, int B, int K, int N, int has_bias, float *dmu_w, float *dvar_w,
                          float *dmu_b, float *dvar_b, void *stream) {
    TAGI_DIMS();
    TAGI_PTR(var_w);
    TAGI_PTR(mu_a);
    TAGI_PTR(dmu_z);
    TAGI_PTR(dvar_z);
    TAGI_PTR(dmu_w);
    TAGI_PTR(dvar_w);
    if (has_bias) {
        TAGI_PTR(var_b);
        TAGI_PTR(dmu_b);
        TAGI_PTR(dvar_b);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc;
    if (pick_tc(__func__, B, K, N, {var_w, mu_a, dmu_z, dvar_z, dmu_w, dvar_w}, &rc)) {
        if (has_bias && linear_bwd_param_tc_fuses_bias(N))  // weight and bias deltas from one kernel
            return linear_bwd_param_tc(var_w, mu_a, dmu_z, dvar_z, B, K, N, dmu_w, dvar_w, st, nullptr, 1, 0, var_b, dmu_b,
                                       dvar_b);
        rc = linear_bwd_param_tc(var_w, mu_a, dmu_z, dvar_z, B, K, N, dmu_w, dvar_w, st);
    } else if (rc == TAGI_OK)
        rc = linear_bwd_param_ffma(var_w, mu_a, dmu_z, dvar_z, B, K, N, dmu_w, dvar_w, st);
    if (rc != TAGI_OK) return rc;
    if (has_bias) rc = linear_bias_delta(var_b, dmu_z, dvar_z, B, N, dmu_b, dvar_b, st);
    return rc;
}

int tagi_linear_bwd_param_rows(const float *var_w, const float *var_b, const float *mu_a, const float *dmu_z,
                               const float *dvar_z, int B, int K, int N, int n0, int n1, int has_bias, float *dmu_w,
                               float *dvar_w, float *dmu_b, float *dvar_b, void *stream) {
    TAGI_DIMS();
    TAGI_REQUIRE(0 <= n0 && n0 < n1 && n1 <= N, "0 <= n0 < n1 <= N required");
    TAGI_PTR(var_w);
    TAGI_PTR(mu_a);
    TAGI_PTR(dmu_z);
    TAGI_PTR(dvar_z);
    TAGI_PTR(dmu_w);
    TAGI_PTR(dvar_w);
    if (has_bias) {
        TAGI_PTR(var_b);
        TAGI_PTR(dmu_b);
        TAGI_PTR(dvar_b);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int Nr = n1 - n0;
    const long w0 = (long)n0 * K;
    var_w += w0, dmu_w += w0, dvar_w += w0, dmu_z += n0, dvar_z += n0;
    int rc = TAGI_OK;
    if (N % 4 != 0 && current_impl() == TAGI_IMPL_TF32X3)
        return fail(TAGI_ERR_UNSUPPORTED, std::string(__func__) + ": TF32X3 needs N (the row pitch of the deltas) to be a "
                                                                  "multiple of 4");
    if (N % 4 == 0 && pick_tc(__func__, B, K, Nr, {var_w, mu_a, dmu_z, dvar_z, dmu_w, dvar_w}, &rc)) {
        if (has_bias && linear_bwd_param_tc_fuses_bias(Nr))
            return linear_bwd_param_tc(var_w, mu_a, dmu_z, dvar_z, B, K, Nr, dmu_w, dvar_w, st, nullptr, 1, N, var_b + n0,
                                       dmu_b + n0, dvar_b + n0);
        rc = linear_bwd_param_tc(var_w, mu_a, dmu_z, dvar_z, B, K, Nr, dmu_w, dvar_w, st, nullptr, 1, N);
    } else if (rc == TAGI_OK || N % 4 != 0)
        rc = linear_bwd_param_ffma(var_w, mu_a, dmu_z, dvar_z, B, K, Nr, dmu_w, dvar_w, st, N);
    if (rc != TAGI_OK) return rc;
    if (has_bias) rc = linear_bias_delta(var_b + n0, dmu_z, dvar_z, B, Nr, dmu_b + n0, dvar_b + n0, st, N);
    return rc;
}

/* ------------------------------------------------------------------ Conv2d */

int tagi_conv2d_out_size(int k, int stride, int wi, int hi, int pad, int pad_type, int *wo, int *ho) {
    TAGI_REQUIRE(wo && ho, "null output pointer");
    TAGI_REQUIRE(k > 0 && stride > 0 && wi > 0 && hi > 0 && pad >= 0, "non-positive kernel, stride or image size");
    int nw, nh;
    if (pad_type == 1) {
        nw = wi - k + 2 * pad, nh = hi - k + 2 * pad;
    } else if (pad_type == 2) {
        nw = wi - k + pad, nh = hi - k + pad;
    } else {
        nw = wi - k, nh = hi - k;
    }
    TAGI_REQUIRE(nw >= 0 && nh >= 0 && nw % stride == 0 && nh % stride == 0,
                 "invalid hyperparameters for conv2d layer: wi=" + std::to_string(wi) + ", hi=" + std::to_string(hi) +
                     ", kernel=" + std::to_string(k) + ", stride=" + std::to_string(stride));
    *wo = nw / stride + 1;
    *ho = nh / stride + 1;
    return TAGI_OK;
}

// true -> run Conv2d on the tensor-core kernels; sets rc when the forced implementation cannot take the layer
static bool pick_conv_tc(const char *who, const tagi_conv2d_geom &g, int pass, std::initializer_list<const void *> ptrs,
                         int *rc) {
    *rc = TAGI_OK;
    const int impl = current_impl();
    if (impl == TAGI_IMPL_FFMA) return false;
    const bool ok = conv_tc_supported(g, pass, ptrs);
    if (impl == TAGI_IMPL_TF32X3) {
        if (!ok)
            *rc = fail(TAGI_ERR_UNSUPPORTED, std::string(who) + ": TF32X3 needs 16-byte aligned tensors and fi*k*k (every "
                                                               "pass), fo (backward passes) and fi (state pass at stride 1) "
                                                               "that are multiples of 4");
        return ok;
    }
    return ok && conv_tc_profitable(g, pass);
}

static int check_geom(const tagi_conv2d_geom *g) {
    TAGI_REQUIRE(g != nullptr, "null geometry");
    TAGI_REQUIRE(g->B > 0 && g->fi > 0 && g->fo > 0, "B, fi and fo must be positive");
    int wo = 0, ho = 0;
    int rc = tagi_conv2d_out_size(g->k, g->stride, g->wi, g->hi, g->pad, g->pad_type, &wo, &ho);
    if (rc != TAGI_OK) return rc;
    TAGI_REQUIRE(wo == g->wo && ho == g->ho, "ho / wo do not match the kernel, stride and padding");
    const long lim = 1L << 31;
    TAGI_REQUIRE((long)g->B * g->fi * g->hi * g->wi < lim && (long)g->B * g->fo * g->ho * g->wo < lim &&
                     (long)g->fo * g->fi * g->k * g->k < lim,
                 "tensor extent exceeds 2^31 elements");
    return TAGI_OK;
}

size_t tagi_conv2d_workspace_bytes(const tagi_conv2d_geom *g) {
    if (check_geom(g) != TAGI_OK) return 0;
    size_t a = conv_tc_workspace_bytes(*g), b = conv_ffma_workspace_bytes(*g);
    const size_t c = conv_param_patch_workspace_bytes(*g), d = conv_pix_patch_workspace_bytes(*g);
    a = a > c ? a : c;
    a = a > d ? a : d;
    // BatchNorm statistics of the layer's output share the block: 16 bytes per channel and 4096-element slice
    const size_t bn = (size_t)g->fo * (((size_t)g->B * g->ho * g->wo + 4095) / 4096) * 16;
    const size_t m = a > b ? a : b;
    return m > bn ? m : bn;
}

int tagi_conv2d_fwd(const tagi_conv2d_geom *g, const float *mu_w, const float *var_w, const float *mu_b,
                    const float *var_b, const float *mu_a, const float *var_a, float *mu_z, float *var_z,
                    void *stream) {
    int rc = check_geom(g);
    if (rc != TAGI_OK) return rc;
    TAGI_PTR(mu_w);
    TAGI_PTR(var_w);
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    TAGI_PTR(mu_z);
    TAGI_PTR(var_z);
    if (g->has_bias) {
        TAGI_PTR(mu_b);
        TAGI_PTR(var_b);
    } else {
        mu_b = var_b = nullptr;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (pick_conv_tc(__func__, *g, CONV_PASS_FWD, {mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_z, var_z}, &rc))
        return conv2d_fwd_tc(*g, mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_z, var_z, st);
    if (rc != TAGI_OK) return rc;
    return conv2d_fwd_ffma(*g, mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_z, var_z, st);
}

int tagi_conv2d_fwd_act(const tagi_conv2d_geom *g, const float *mu_w, const float *var_w, const float *mu_b,
                        const float *var_b, const float *mu_a, const float *var_a, int act, float *mu_a_out,
                        float *var_a_out, float *jcb_out, void *stream) {
    int rc = check_geom(g);
    if (rc != TAGI_OK) return rc;
    TAGI_REQUIRE(act == TAGI_ACT_RELU || act == TAGI_ACT_MIXTURE_RELU, "unknown activation id");
    TAGI_PTR(mu_w);
    TAGI_PTR(var_w);
    TAGI_PTR(mu_a);
    TAGI_PTR(var_a);
    TAGI_PTR(mu_a_out);
    TAGI_PTR(var_a_out);
    TAGI_PTR(jcb_out);
    if (g->has_bias) {
        TAGI_PTR(mu_b);
        TAGI_PTR(var_b);
    } else {
        mu_b = var_b = nullptr;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (pick_conv_tc(__func__, *g, CONV_PASS_FWD, {mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_a_out, var_a_out, jcb_out},
                     &rc) &&
        conv2d_fwd_tc_fuses_relu(*g) && act == TAGI_ACT_RELU)
        return conv2d_fwd_tc(*g, mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_a_out, var_a_out, st, jcb_out);
    if (rc != TAGI_OK) return rc;
    rc = tagi_conv2d_fwd(g, mu_w, var_w, mu_b, var_b, mu_a, var_a, mu_a_out, var_a_out, stream);
    if (rc != TAGI_OK) return rc;
    return act_after(act, mu_a_out, var_a_out, (size_t)g->B * g->fo * g->ho * g->wo, jcb_out, stream);
}

int tagi_conv2d_fwd_relu(const tagi_conv2d_geom *g, const float *mu_w, const float *var_w, const float *mu_b,
                         const float *var_b, const float *mu_a, const float *var_a, float *mu_a_out, float *var_a_out,
                         float *jcb_out, void *stream) {
    return tagi_conv2d_fwd_act(g, mu_w, var_w, mu_b, var_b, mu_a, var_a, TAGI_ACT_RELU, mu_a_out, var_a_out, jcb_out, stream);
}

int tagi_conv2d_bwd_state(const tagi_conv2d_geom *g, const float *mu_w, const float *jcb, const float *dmu_z,
                          const float *dvar_z, float *dmu_a, float *dvar_a, void *stream) {
    int rc = check_geom(g);
    if (rc != TAGI_OK) return rc;
    TAGI_PTR(mu_w);
    if (jcb) TAGI_PTR(jcb);
    TAGI_PTR(dmu_z);
    TAGI_PTR(dvar_z);
    TAGI_PTR(dmu_a);
    TAGI_PTR(dvar_a);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (pick_conv_tc(__func__, *g, CONV_PASS_STATE, {mu_w, jcb, dmu_z, dvar_z, dmu_a, dvar_a}, &rc))
        return conv2d_bwd_state_tc(*g, mu_w, jcb, dmu_z, dvar_z, dmu_a, dvar_a, st);
    if (rc != TAGI_OK) return rc;
    return conv2d_bwd_state_ffma(*g, mu_w, jcb, dmu_z, dvar_z, dmu_a, dvar_a, st);
}

int tagi_conv2d_bwd_param(const tagi_conv2d_geom *g, const float *var_w, const float *var_b, const float *mu_a,
                          const float *dmu_z, const float *dvar_z, float *dmu_w, float *dvar_w, float *dmu_b,
                          float *dvar_b, void *stream) {
    int rc = check_geom(g);
    if (rc != TAGI_OK) return rc;
    TAGI_PTR(var_w);
    TAGI_PTR(mu_a);
    TAGI_PTR(dmu_z);
    TAGI_PTR(dvar_z);
    TAGI_PTR(dmu_w);
    TAGI_PTR(dvar_w);
    if (g->has_bias) {
        TAGI_PTR(var_b);
        TAGI_PTR(dmu_b);
        TAGI_PTR(dvar_b);
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Implicit GEMM on the tensor cores where the tensors can be read by TMA as they lie (image widths multiples of 4):
    // no im2col matrix, no regrouped deltas. TAGI_B200_CONV_PARAM=explicit keeps the gather passes (for comparison).
    static const bool explicit_param = [] {
        const char *e = std::getenv("TAGI_B200_CONV_PARAM");
        return e && !std::strcmp(e, "explicit");
    }();
    if (current_impl() != TAGI_IMPL_FFMA && !explicit_param && (long)g->B * g->ho * g->wo >= 1024 &&
        conv_param_patch_supported(*g, {var_w, mu_a, dmu_z, dvar_z, dmu_w, dvar_w})) {
        rc = conv2d_bwd_param_patch(*g, var_w, mu_a, dmu_z, dvar_z, dmu_w, dvar_w, st);
        if (rc == TAGI_OK && g->has_bias) rc = conv_bias_delta(*g, var_b, dmu_z, dvar_z, dmu_b, dvar_b, st);
        return rc;
    }
    if (pick_conv_tc(__func__, *g, CONV_PASS_PARAM, {var_w, mu_a, dmu_z, dvar_z, dmu_w, dvar_w}, &rc)) {
        rc = conv2d_bwd_param_tc(*g, var_w, mu_a, dmu_z, dvar_z, dmu_w, dvar_w, st);
        if (rc == TAGI_OK && g->has_bias) rc = conv_bias_delta(*g, var_b, dmu_z, dvar_z, dmu_b, dvar_b, st);
        return rc;
    }
    if (rc != TAGI_OK) return rc;
    return conv2d_bwd_param_ffma(*g, var_w, var_b, mu_a, dmu_z, dvar_z, dmu_w, dvar_w, dmu_b, dvar_b, st);
}

int tagi_conv2d_bwd_param_noalloc(const tagi_conv2d_geom *g, const float *var_w, const float *var_b, const float *mu_a,
                                  const float *dmu_z, const float *dvar_z, float *dmu_w, float *dvar_w, float *dmu_b,
                                  float *dvar_b, void *stream) {
    int rc = check_geom(g);
    if (rc != TAGI_OK) return rc;
    TAGI_PTR(var_w);
    TAGI_PTR(mu_a);
    TAGI_PTR(dmu_z);
    TAGI_PTR(dvar_z);
    TAGI_PTR(dmu_w);
    TAGI_PTR(dvar_w);
    if (g->has_bias) {
        TAGI_PTR(var_b);
        TAGI_PTR(dmu_b);
        TAGI_PTR(dvar_b);
    }
    return conv2d_bwd_param_noalloc(*g, var_w, var_b, mu_a, dmu_z, dvar_z, dmu_w, dvar_w, dmu_b, dvar_b,
                                    static_cast<cudaStream_t>(stream));
}

}  // extern "C"
