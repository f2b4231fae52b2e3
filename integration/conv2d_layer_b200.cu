// Drop-in implementation of cuTAGI's `Conv2dCuda` (declared in include/conv2d_layer_cuda.cuh:5-73 of the cuTAGI tree)
// on top of libtagi_b200's C ABI, linked into the cuTAGI library in place of src/conv2d_layer_cuda.cu. The kernels
// compute the receptive-field gather from the geometry, so the three index tables of the original (and their device
// copies), the Jacobian permute and the delta permute (src/conv2d_layer_cuda.cu:292-345, 163-172, 504-511) are not
// built; the members that hold them stay empty and temp_states is not touched.
#include "conv2d_layer_cuda.cuh"

#include "conv2d_layer.h"
#include "custom_logger.h"
#include "param_init.h"
#include "ddp_b200_hooks.h"
#include "tagi_b200.h"

namespace {
void require_ok(int status) {
    if (status != TAGI_OK) LOG(LogLevel::ERROR, std::string("tagi_b200: ") + tagi_last_error_string());
}
}  // namespace

Conv2dCuda::Conv2dCuda(size_t in_channels, size_t out_channels, size_t kernel_size, bool bias, int stride, int padding,
                       int padding_type, size_t in_width, size_t in_height, float gain_w, float gain_b,
                       std::string init_method, int device_idx)
    : gain_w(gain_w), gain_b(gain_b), init_method(init_method), kernel_size(kernel_size), padding(padding),
      stride(stride), padding_type(padding_type), d_idx_mwa_2(nullptr), d_idx_cov_zwa_1(nullptr),
      d_idx_var_z_ud(nullptr) {
    this->in_width = in_width;
    this->in_height = in_height;
    this->in_channels = in_channels;
    this->out_channels = out_channels;
    this->bias = bias;
    this->device_idx = device_idx;
}

Conv2dCuda::~Conv2dCuda() = default;

std::string Conv2dCuda::get_layer_info() const {
    return "Conv2d(" + std::to_string(in_channels) + "," + std::to_string(out_channels) + "," +
           std::to_string(out_width) + "," + std::to_string(out_height) + "," + std::to_string(kernel_size) + ")";
}
std::string Conv2dCuda::get_layer_name() const { return "Conv2dCuda"; }
LayerType Conv2dCuda::get_layer_type() const { return LayerType::Conv2d; }

void Conv2dCuda::compute_input_output_size(const InitArgs &args) {
    if (in_height == 0 || in_width == 0) {
        in_width = args.width;
        in_height = args.height;
    }
    int wo = 0, ho = 0;
    // same rule and same message as compute_downsample_img_size_v2 (src/conv2d_layer.cpp:581-628)
    require_ok(tagi_conv2d_out_size(static_cast<int>(kernel_size), stride, static_cast<int>(in_width),
                                    static_cast<int>(in_height), padding, padding_type, &wo, &ho));
    out_width = wo;
    out_height = ho;
    input_size = in_width * in_width * in_channels;  // square images, as in the CPU class
    output_size = out_width * out_height * out_channels;
}

void Conv2dCuda::get_number_param() {
    num_weights = kernel_size * kernel_size * in_channels * out_channels;
    num_biases = bias ? out_channels : 0;
}

void Conv2dCuda::init_weight_bias() {
    std::tie(mu_w, var_w, mu_b, var_b) = init_weight_bias_conv2d(kernel_size, in_channels, out_channels, init_method,
                                                                 gain_w, gain_b, num_weights, num_biases);
    allocate_param_memory();
    params_to_device();
}

void Conv2dCuda::allocate_conv_index() {}
void Conv2dCuda::conv_index_to_device() {}
void Conv2dCuda::lazy_index_init() {}

void Conv2dCuda::preinit_layer() {
    if (num_weights == 0) {
        get_number_param();
        init_weight_bias();
        if (training) allocate_param_delta();
    }
}

void Conv2dCuda::to(int device_idx_) { device_idx = device_idx_; }

namespace {
tagi_conv2d_geom geometry_of(const Conv2dCuda &l, int batch) {
    tagi_conv2d_geom g;
    g.B = batch;
    g.fi = static_cast<int>(l.in_channels);
    g.hi = static_cast<int>(l.in_height);
    g.wi = static_cast<int>(l.in_width);
    g.fo = static_cast<int>(l.out_channels);
    g.ho = static_cast<int>(l.out_height);
    g.wo = static_cast<int>(l.out_width);
    g.k = static_cast<int>(l.kernel_size);
    g.stride = l.stride;
    g.pad = l.padding;
    g.pad_type = l.padding_type;
    g.has_bias = l.bias ? 1 : 0;
    return g;
}
}  // namespace

void Conv2dCuda::forward(BaseHiddenStates &input_states, BaseHiddenStates &output_states, BaseTempStates &) {
    auto *in = dynamic_cast<HiddenStateCuda *>(&input_states);
    auto *out = dynamic_cast<HiddenStateCuda *>(&output_states);
    if (input_size != input_states.actual_size)
        LOG(LogLevel::ERROR, "Input size mismatch: " + std::to_string(input_size) + " vs " +
                                 std::to_string(input_states.actual_size));
    const int batch = static_cast<int>(input_states.block_size);
    set_cap_factor_udapte(batch);
    preinit_layer();  // parameters are created on the first forward, as in the original

    output_states.width = out_width;
    output_states.height = out_height;
    output_states.depth = out_channels;
    output_states.block_size = batch;
    output_states.actual_size = output_size;

    const tagi_conv2d_geom g = geometry_of(*this, batch);
    // the library's scratch block is sized here for all three passes of this layer, so that the backward pass never
    // allocates (a no-op once the block is large enough)
    if (training) require_ok(tagi_reserve_scratch(tagi_conv2d_workspace_bytes(&g)));
    require_ok(tagi_conv2d_fwd(&g, d_mu_w, d_var_w, d_mu_b, d_var_b, in->d_mu_a, in->d_var_a, out->d_mu_a, out->d_var_a,
                               nullptr));
    if (training) store_states_for_training_cuda(*in, *out);
}

void Conv2dCuda::backward(BaseDeltaStates &input_delta_states, BaseDeltaStates &output_delta_states, BaseTempStates &,
                          bool state_udapte) {
    auto *saved = dynamic_cast<BackwardStateCuda *>(bwd_states.get());
    auto *din = dynamic_cast<DeltaStateCuda *>(&input_delta_states);
    auto *dout = dynamic_cast<DeltaStateCuda *>(&output_delta_states);
    const tagi_conv2d_geom g = geometry_of(*this, static_cast<int>(input_delta_states.block_size));
    // parameters first, then states: the state pass overwrites the buffer the deltas may share in LayerBlock
    if (param_update) {
        require_ok(tagi_conv2d_bwd_param(&g, d_var_w, d_var_b, saved->d_mu_a, din->d_delta_mu, din->d_delta_var,
                                         d_delta_mu_w, d_delta_var_w, d_delta_mu_b, d_delta_var_b, nullptr));
        // data-parallel runs: this layer's deltas may be exchanged from now on (no effect without a DDPSequential)
        ddp_b200_deltas_ready(d_delta_mu_w);
        ddp_b200_deltas_ready(d_delta_var_w);
        if (bias) {
            ddp_b200_deltas_ready(d_delta_mu_b);
            ddp_b200_deltas_ready(d_delta_var_b);
        }
    }
    if (state_udapte)
        require_ok(tagi_conv2d_bwd_state(&g, d_mu_w, saved->d_jcb, din->d_delta_mu, din->d_delta_var, dout->d_delta_mu,
                                         dout->d_delta_var, nullptr));
}

std::unique_ptr<BaseLayer> Conv2dCuda::to_host() {
    tagi_b200_raise_on_kernel_abort();  // this call synchronises anyway: report an aborted tensor-core launch here
    auto host = std::make_unique<Conv2d>(in_channels, out_channels, kernel_size, bias, stride, padding, padding_type,
                                         in_width, in_height, gain_w, gain_b, init_method);
    host->mu_w = mu_w;
    host->var_w = var_w;
    host->mu_b = mu_b;
    host->var_b = var_b;
    return host;
}
