// C-ABI door onto the reference's own CPU classes (test infrastructure only).
//
// This translation unit is compiled by oracle/Makefile against the reference's
// headers and linked with object files built from the reference's own sources
// (src/linear_layer.cpp, src/conv2d_layer.cpp, src/base_layer.cpp, ...), which
// stay where they are. It drives `Linear` (include/linear_layer.h:99-141),
// `Conv2d` (include/conv2d_layer.h:20-81), `BatchNorm2d`
// (include/batchnorm_layer.h:8-64) and `AvgPool2d` (include/pooling_layer.h:13-70) exactly the way `Sequential` does
// (src/sequential.cpp:323-331, 392-410): hidden/delta/temp state objects in,
// `forward` / `backward` virtual calls, results read from the state objects and
// from the layer's `delta_*` members. Nothing here restates any arithmetic.
//
// Every function returns 0 on success and -1 when the reference raised
// (LOG(ERROR) throws std::runtime_error, src/custom_logger.cpp:58-60); the
// message is kept for tagi_ref_last_error().
#include <cstring>
#include <exception>
#include <string>
#include <vector>

#include "base_layer.h"
#include "conv2d_layer.h"
#include "data_struct.h"
#include "linear_layer.h"
#include "activation.h"
#include "batchnorm_layer.h"
#include "pooling_layer.h"

namespace {
std::string g_err;

std::vector<float> vec(const float *p, size_t n) {
    return p ? std::vector<float>(p, p + n) : std::vector<float>(n, 0.0f);
}
void out(float *dst, const std::vector<float> &v, size_t n) {
    if (dst) std::memcpy(dst, v.data(), n * sizeof(float));
}

void set_params(BaseLayer &l, size_t nw, size_t nb, const float *mu_w,
                const float *var_w, const float *mu_b, const float *var_b) {
    l.mu_w = vec(mu_w, nw);
    l.var_w = vec(var_w, nw);
    l.mu_b = vec(mu_b, nb);
    l.var_b = vec(var_b, nb);
    l.num_weights = nw;
    l.num_biases = nb;
    l.allocate_param_delta();
}

template <class F>
int guarded(F &&f) {
    try {
        f();
        return 0;
    } catch (const std::exception &e) {
        g_err = e.what();
    } catch (...) {
        g_err = "unknown exception";
    }
    return -1;
}
}  // namespace

extern "C" {

const char *tagi_ref_last_error() { return g_err.c_str(); }

// Linear::forward (src/linear_layer.cpp:524-572)
int tagi_ref_linear_forward(int B, int K, int N, int has_bias, int threads,
                            const float *mu_w, const float *var_w,
                            const float *mu_b, const float *var_b,
                            const float *mu_a, const float *var_a, float *mu_z,
                            float *var_z) {
    return guarded([&] {
        Linear layer(K, N, has_bias != 0);
        set_params(layer, (size_t)K * N, has_bias ? N : 0, mu_w, var_w, mu_b,
                   var_b);
        layer.set_threads(threads);
        size_t cap = (size_t)B * (K > N ? K : N);
        BaseHiddenStates in(cap, B), outs(cap, B);
        BaseTempStates tmp(cap, B);
        std::memcpy(in.mu_a.data(), mu_a, sizeof(float) * B * K);
        std::memcpy(in.var_a.data(), var_a, sizeof(float) * B * K);
        in.block_size = B;
        in.actual_size = K;
        layer.forward(in, outs, tmp);
        out(mu_z, outs.mu_a, (size_t)B * N);
        out(var_z, outs.var_a, (size_t)B * N);
    });
}

// Linear::backward (src/linear_layer.cpp:574-631). `mu_a` and `jcb` are what
// the forward pass saved in bwd_states (src/base_layer.cpp:212-228).
int tagi_ref_linear_backward(int B, int K, int N, int has_bias, int threads,
                             int state_update, const float *mu_w,
                             const float *var_w, const float *var_b,
                             const float *mu_a, const float *jcb,
                             const float *dmu_z, const float *dvar_z,
                             float *dmu_a, float *dvar_a, float *dmu_w,
                             float *dvar_w, float *dmu_b, float *dvar_b) {
    return guarded([&] {
        Linear layer(K, N, has_bias != 0);
        set_params(layer, (size_t)K * N, has_bias ? N : 0, mu_w, var_w, nullptr,
                   var_b);
        layer.set_threads(threads);
        layer.bwd_states->set_size((size_t)B * K);
        std::memcpy(layer.bwd_states->mu_a.data(), mu_a, sizeof(float) * B * K);
        std::memcpy(layer.bwd_states->jcb.data(), jcb, sizeof(float) * B * K);
        size_t cap = (size_t)B * (K > N ? K : N);
        BaseDeltaStates din(cap, B), dout(cap, B);
        BaseTempStates tmp(cap, B);
        std::memcpy(din.delta_mu.data(), dmu_z, sizeof(float) * B * N);
        std::memcpy(din.delta_var.data(), dvar_z, sizeof(float) * B * N);
        din.block_size = B;
        din.actual_size = N;
        layer.backward(din, dout, tmp, state_update != 0);
        if (state_update) {
            out(dmu_a, dout.delta_mu, (size_t)B * K);
            out(dvar_a, dout.delta_var, (size_t)B * K);
        }
        out(dmu_w, layer.delta_mu_w, (size_t)K * N);
        out(dvar_w, layer.delta_var_w, (size_t)K * N);
        if (has_bias) {
            out(dmu_b, layer.delta_mu_b, N);
            out(dvar_b, layer.delta_var_b, N);
        }
    });
}

// Output geometry as Conv2d::compute_input_output_size sees it
// (src/conv2d_layer.cpp:48-65, 581-628). Raises for non-divisible strides.
int tagi_ref_conv2d_out_size(int k, int stride, int wi, int hi, int pad,
                             int pad_type, int *wo, int *ho) {
    return guarded([&] {
        int w = 0, h = 0;
        std::tie(w, h) =
            compute_downsample_img_size_v2(k, stride, wi, hi, pad, pad_type);
        *wo = w;
        *ho = h;
    });
}

static std::unique_ptr<Conv2d> make_conv(int fi, int fo, int k, int has_bias,
                                         int stride, int pad, int pad_type,
                                         int wi, int hi, int threads) {
    auto layer = std::make_unique<Conv2d>(fi, fo, k, has_bias != 0, stride, pad,
                                          pad_type, wi, hi);
    InitArgs args(wi, hi, fi);
    layer->compute_input_output_size(args);
    layer->get_number_param();
    layer->set_threads(threads);
    return layer;
}

// Conv2d::forward (src/conv2d_layer.cpp:117-175); index tables are built by the
// reference itself on this first call (lazy_index_init, :96-115).
int tagi_ref_conv2d_forward(int B, int fi, int hi, int wi, int fo, int k,
                            int stride, int pad, int pad_type, int has_bias,
                            int threads, const float *mu_w, const float *var_w,
                            const float *mu_b, const float *var_b,
                            const float *mu_a, const float *var_a, float *mu_z,
                            float *var_z) {
    return guarded([&] {
        auto layer =
            make_conv(fi, fo, k, has_bias, stride, pad, pad_type, wi, hi, threads);
        set_params(*layer, layer->num_weights, layer->num_biases, mu_w, var_w,
                   mu_b, var_b);
        size_t n_in = (size_t)fi * hi * wi, n_out = layer->output_size;
        size_t cap = (size_t)B * (n_in > n_out ? n_in : n_out);
        BaseHiddenStates in(cap, B), outs(cap, B);
        BaseTempStates tmp(cap, B);
        std::memcpy(in.mu_a.data(), mu_a, sizeof(float) * B * n_in);
        std::memcpy(in.var_a.data(), var_a, sizeof(float) * B * n_in);
        in.block_size = B;
        in.actual_size = layer->input_size;
        layer->forward(in, outs, tmp);
        out(mu_z, outs.mu_a, (size_t)B * n_out);
        out(var_z, outs.var_a, (size_t)B * n_out);
    });
}

// Conv2d::backward (src/conv2d_layer.cpp:177-246), permutes included.
int tagi_ref_conv2d_backward(int B, int fi, int hi, int wi, int fo, int k,
                             int stride, int pad, int pad_type, int has_bias,
                             int threads, int state_update, const float *mu_w,
                             const float *var_w, const float *var_b,
                             const float *mu_a, const float *jcb,
                             const float *dmu_z, const float *dvar_z,
                             float *dmu_a, float *dvar_a, float *dmu_w,
                             float *dvar_w, float *dmu_b, float *dvar_b) {
    return guarded([&] {
        auto layer =
            make_conv(fi, fo, k, has_bias, stride, pad, pad_type, wi, hi, threads);
        set_params(*layer, layer->num_weights, layer->num_biases, mu_w, var_w,
                   nullptr, var_b);
        size_t n_in = (size_t)fi * hi * wi, n_out = layer->output_size;
        size_t cap = (size_t)B * (n_in > n_out ? n_in : n_out);
        // a forward on zeros makes the layer build its index tables and size
        // its saved-state vectors; the saved states are then overwritten
        {
            BaseHiddenStates in(cap, B), outs(cap, B);
            BaseTempStates tmp(cap, B);
            in.block_size = B;
            in.actual_size = layer->input_size;
            layer->forward(in, outs, tmp);
        }
        std::memcpy(layer->bwd_states->mu_a.data(), mu_a,
                    sizeof(float) * B * n_in);
        std::memcpy(layer->bwd_states->jcb.data(), jcb, sizeof(float) * B * n_in);
        BaseDeltaStates din(cap, B), dout(cap, B);
        BaseTempStates tmp(cap, B);
        std::memcpy(din.delta_mu.data(), dmu_z, sizeof(float) * B * n_out);
        std::memcpy(din.delta_var.data(), dvar_z, sizeof(float) * B * n_out);
        din.block_size = B;
        din.actual_size = n_out;
        layer->backward(din, dout, tmp, state_update != 0);
        if (state_update) {
            out(dmu_a, dout.delta_mu, (size_t)B * n_in);
            out(dvar_a, dout.delta_var, (size_t)B * n_in);
        }
        out(dmu_w, layer->delta_mu_w, layer->num_weights);
        out(dvar_w, layer->delta_var_w, layer->num_weights);
        if (has_bias) {
            out(dmu_b, layer->delta_mu_b, fo);
            out(dvar_b, layer->delta_var_b, fo);
        }
    });
}

// BaseLayer::update_weights / update_biases (src/base_layer.cpp:116-162) with
// the cap factor chosen from the batch size (:164-187). Updates in place and
// returns the count of variances that were reset in *neg_var.
int tagi_ref_param_update(int batch_size, size_t nw, size_t nb, float *mu_w,
                          float *var_w, float *mu_b, float *var_b,
                          const float *dmu_w, const float *dvar_w,
                          const float *dmu_b, const float *dvar_b,
                          int *neg_var) {
    return guarded([&] {
        BaseLayer l;
        l.bias = nb > 0;
        set_params(l, nw, nb, mu_w, var_w, mu_b, var_b);
        l.delta_mu_w = vec(dmu_w, nw);
        l.delta_var_w = vec(dvar_w, nw);
        l.delta_mu_b = vec(dmu_b, nb);
        l.delta_var_b = vec(dvar_b, nb);
        l.set_cap_factor_udapte(batch_size);
        l.update_weights();
        l.update_biases();
        out(mu_w, l.mu_w, nw);
        out(var_w, l.var_w, nw);
        out(mu_b, l.mu_b, nb);
        out(var_b, l.var_b, nb);
        if (neg_var) *neg_var = l.neg_var_w_counter;
    });
}

// BatchNorm2d::forward in training mode (src/batchnorm_layer.cpp:849-985): batch statistics, running averages
// (mu_ra / var_ra in, updated out; `first_batch` selects momentum 0 as the reference does), normalisation.
int tagi_ref_bn2d_forward(int B, int C, int hi, int wi, int has_bias, int threads, int training, int first_batch,
                          float eps, float momentum, const float *mu_w, const float *var_w, const float *mu_b,
                          const float *var_b, const float *mu_a, const float *var_a, float *mu_ra, float *var_ra,
                          float *mu_batch, float *var_batch, float *mu_z, float *var_z) {
    return guarded([&] {
        BatchNorm2d layer(C, eps, momentum, has_bias != 0);
        set_params(layer, C, has_bias ? C : 0, mu_w, var_w, mu_b, var_b);
        InitArgs args(wi, hi, C);
        layer.compute_input_output_size(args);
        layer.set_threads(threads);
        layer.training = training != 0;
        layer.first_batch = first_batch != 0;
        layer.mu_ra = vec(mu_ra, C);
        layer.var_ra = vec(var_ra, C);
        size_t n = (size_t)C * hi * wi, cap = (size_t)B * n;
        BaseHiddenStates in(cap, B), outs(cap, B);
        BaseTempStates tmp(cap, B);
        std::memcpy(in.mu_a.data(), mu_a, sizeof(float) * cap);
        std::memcpy(in.var_a.data(), var_a, sizeof(float) * cap);
        in.block_size = B;
        in.actual_size = n;
        layer.forward(in, outs, tmp);
        out(mu_z, outs.mu_a, cap);
        out(var_z, outs.var_a, cap);
        out(mu_ra, layer.mu_ra, C);
        out(var_ra, layer.var_ra, C);
        out(mu_batch, layer.mu_norm_batch, C);
        out(var_batch, layer.var_norm_batch, C);
    });
}

// BatchNorm2d::backward (src/batchnorm_layer.cpp:987-1129); mu_a / jcb are the saved input states, mu_batch / var_batch
// the batch statistics of the forward pass.
int tagi_ref_bn2d_backward(int B, int C, int hi, int wi, int has_bias, int threads, float eps, const float *mu_w,
                           const float *var_w, const float *var_b, const float *mu_a, const float *jcb,
                           const float *mu_batch, const float *var_batch, const float *dmu_o, const float *dvar_o,
                           float *dmu, float *dvar, float *dmu_w, float *dvar_w, float *dmu_b, float *dvar_b) {
    return guarded([&] {
        BatchNorm2d layer(C, eps, 0.9f, has_bias != 0);
        set_params(layer, C, has_bias ? C : 0, mu_w, var_w, nullptr, var_b);
        InitArgs args(wi, hi, C);
        layer.compute_input_output_size(args);
        layer.set_threads(threads);
        layer.mu_norm_batch = vec(mu_batch, C);
        layer.var_norm_batch = vec(var_batch, C);
        size_t n = (size_t)C * hi * wi, cap = (size_t)B * n;
        layer.input_size = layer.output_size = n;
        layer.bwd_states->set_size(cap);
        std::memcpy(layer.bwd_states->mu_a.data(), mu_a, sizeof(float) * cap);
        std::memcpy(layer.bwd_states->jcb.data(), jcb, sizeof(float) * cap);
        BaseDeltaStates din(cap, B), dout(cap, B);
        BaseTempStates tmp(cap, B);
        std::memcpy(din.delta_mu.data(), dmu_o, sizeof(float) * cap);
        std::memcpy(din.delta_var.data(), dvar_o, sizeof(float) * cap);
        din.block_size = B;
        din.actual_size = n;
        layer.backward(din, dout, tmp, true);
        out(dmu, dout.delta_mu, cap);
        out(dvar, dout.delta_var, cap);
        out(dmu_w, layer.delta_mu_w, C);
        out(dvar_w, layer.delta_var_w, C);
        if (has_bias) {
            out(dmu_b, layer.delta_mu_b, C);
            out(dvar_b, layer.delta_var_b, C);
        }
    });
}

// AvgPool2d::forward / backward (src/pooling_layer.cpp:59-176); index tables built by the reference itself.
int tagi_ref_avgpool2d(int B, int C, int hi, int wi, int k, int stride, int pad, int pad_type, int threads,
                       const float *mu_a, const float *var_a, const float *jcb, const float *dmu_o,
                       const float *dvar_o, int *wo, int *ho, float *mu_z, float *var_z, float *dmu, float *dvar) {
    return guarded([&] {
        AvgPool2d layer(k, stride, pad, pad_type);
        InitArgs args(wi, hi, C);
        layer.compute_input_output_size(args);
        layer.set_threads(threads);
        *wo = layer.out_width;
        *ho = layer.out_height;
        size_t n_in = (size_t)C * hi * wi, n_out = layer.output_size;
        size_t cap = (size_t)B * (n_in > n_out ? n_in : n_out);
        BaseHiddenStates in(cap, B), outs(cap, B);
        BaseTempStates tmp(cap, B);
        std::memcpy(in.mu_a.data(), mu_a, sizeof(float) * B * n_in);
        std::memcpy(in.var_a.data(), var_a, sizeof(float) * B * n_in);
        in.block_size = B;
        in.actual_size = n_in;
        layer.forward(in, outs, tmp);
        out(mu_z, outs.mu_a, (size_t)B * n_out);
        out(var_z, outs.var_a, (size_t)B * n_out);
        if (!dmu_o) return;
        std::memcpy(layer.bwd_states->jcb.data(), jcb, sizeof(float) * B * n_in);
        BaseDeltaStates din(cap, B), dout(cap, B);
        std::memcpy(din.delta_mu.data(), dmu_o, sizeof(float) * B * n_out);
        std::memcpy(din.delta_var.data(), dvar_o, sizeof(float) * B * n_out);
        din.block_size = B;
        din.actual_size = n_out;
        layer.backward(din, dout, tmp, true);
        out(dmu, dout.delta_mu, (size_t)B * n_in);
        out(dvar, dout.delta_var, (size_t)B * n_in);
    });
}

// mixture_relu_mean_var (src/activation.cpp:152-178), the CPU kernel behind MixtureReLU::forward (:724-744)
int tagi_ref_mixture_relu(size_t n, const float *mu_z, const float *var_z, float *mu_a, float *var_a, float *jcb) {
    return guarded([&] {
        std::vector<float> mz = vec(mu_z, n), vz = vec(var_z, n), ma(n), va(n), j(n);
        mixture_relu_mean_var(mz, vz, 0, (int)n, ma, j, va);
        out(mu_a, ma, n);
        out(var_a, va, n);
        out(jcb, j, n);
    });
}

}  // extern "C"
