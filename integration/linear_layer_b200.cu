// Drop-in implementation of cuTAGI's `LinearCuda` (declared in include/linear_layer_cuda.cuh:54-96 of the cuTAGI
// tree) on top of libtagi_b200's C ABI. Compiled against the cuTAGI headers and linked into the cuTAGI library in
// place of src/linear_layer_cuda.cu; every other cuTAGI class (Sequential, the state containers, the bindings) is
// used unchanged. The three launcher calls of the original (src/linear_layer_cuda.cu:12,75,123,316) become
// tagi_linear_fwd / tagi_linear_bwd_state / tagi_linear_bwd_param.
#include "linear_layer_cuda.cuh"

#include "custom_logger.h"
#include "linear_layer.h"
#include "param_init.h"
#include "ddp_b200_hooks.h"
#include "tagi_b200.h"

namespace {
// cuTAGI reports errors by LOG(ERROR), which throws std::runtime_error (src/custom_logger.cpp:58-60)
void require_ok(int status) {
    if (status != TAGI_OK) LOG(LogLevel::ERROR, std::string("tagi_b200: ") + tagi_last_error_string());
}
}  // namespace

LinearCuda::LinearCuda(size_t ip_size, size_t op_size, bool bias, float gain_weight, float gain_bias,
                       std::string method, int device_idx)
    : gain_w(gain_weight), gain_b(gain_bias), init_method(method) {
    input_size = ip_size;
    output_size = op_size;
    this->bias = bias;
    this->device_idx = device_idx;
    num_weights = ip_size * op_size;
    num_biases = bias ? op_size : 0;
    if (training) allocate_param_delta();
}

LinearCuda::~LinearCuda() = default;

std::string LinearCuda::get_layer_info() const {
    return "Linear(" + std::to_string(input_size) + "," + std::to_string(output_size) + ")";
}
std::string LinearCuda::get_layer_name() const { return "LinearCuda"; }
LayerType LinearCuda::get_layer_type() const { return LayerType::Linear; }

void LinearCuda::init_weight_bias() {
    std::tie(mu_w, var_w, mu_b, var_b) =
        init_weight_bias_linear(init_method, gain_w, gain_b, input_size, output_size, num_weights, num_biases);
    allocate_param_memory();
    params_to_device();
}

void LinearCuda::forward(BaseHiddenStates &input_states, BaseHiddenStates &output_states, BaseTempStates &) {
    auto *in = dynamic_cast<HiddenStateCuda *>(&input_states);
    auto *out = dynamic_cast<HiddenStateCuda *>(&output_states);
    if (input_size != input_states.actual_size)
        LOG(LogLevel::ERROR, "Input size mismatch: " + std::to_string(input_size) + " vs " +
                                 std::to_string(input_states.actual_size));
    const int batch = static_cast<int>(input_states.block_size);
    set_cap_factor_udapte(batch);
    require_ok(tagi_linear_fwd(d_mu_w, d_var_w, d_mu_b, d_var_b, in->d_mu_a, in->d_var_a, batch,
                               static_cast<int>(input_size), static_cast<int>(output_size), bias ? 1 : 0, out->d_mu_a,
                               out->d_var_a, nullptr));
    output_states.block_size = batch;
    output_states.actual_size = output_size;
    if (training) store_states_for_training_cuda(*in, *out);
}

void LinearCuda::backward(BaseDeltaStates &input_delta_states, BaseDeltaStates &output_delta_states, BaseTempStates &,
                          bool state_udapte) {
    auto *saved = dynamic_cast<BackwardStateCuda *>(bwd_states.get());
    auto *din = dynamic_cast<DeltaStateCuda *>(&input_delta_states);
    auto *dout = dynamic_cast<DeltaStateCuda *>(&output_delta_states);
    const int batch = static_cast<int>(input_delta_states.block_size);
    const int k = static_cast<int>(input_size), n = static_cast<int>(output_size);
    if (state_udapte)
        require_ok(tagi_linear_bwd_state(d_mu_w, saved->d_jcb, din->d_delta_mu, din->d_delta_var, batch, k, n,
                                         dout->d_delta_mu, dout->d_delta_var, nullptr));
    if (param_update) {
        require_ok(tagi_linear_bwd_param(d_var_w, d_var_b, saved->d_mu_a, din->d_delta_mu, din->d_delta_var, batch, k,
                                         n, bias ? 1 : 0, d_delta_mu_w, d_delta_var_w, d_delta_mu_b, d_delta_var_b,
                                         nullptr));
        // data-parallel runs: this layer's deltas may be exchanged from now on (no effect without a DDPSequential)
        ddp_b200_deltas_ready(d_delta_mu_w);
        ddp_b200_deltas_ready(d_delta_var_w);
        if (bias) {
            ddp_b200_deltas_ready(d_delta_mu_b);
            ddp_b200_deltas_ready(d_delta_var_b);
        }
    }
}

std::unique_ptr<BaseLayer> LinearCuda::to_host() {
    tagi_b200_raise_on_kernel_abort();  // this call synchronises anyway: report an aborted tensor-core launch here
    auto host = std::make_unique<Linear>(input_size, output_size, bias, gain_w, gain_b, init_method);
    host->mu_w = mu_w;
    host->var_w = var_w;
    host->mu_b = mu_b;
    host->var_b = var_b;
    return host;
}
