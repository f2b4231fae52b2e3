// Drop-in bodies for the hot methods of cuTAGI's layers that sit between the Linear / Conv2d calls of a CNN or ResNet
// step, on libtagi_b200's C ABI:
//   BatchNorm2dCuda::forward / backward   (src/batchnorm_layer_cuda.cu:832-1087)  -> tagi_bn2d_fwd / tagi_bn2d_bwd
//   AvgPool2dCuda::forward / backward     (src/pooling_layer_cuda.cu:167-270)     -> tagi_avgpool2d_fwd / _bwd_state
//   ReLUCuda::forward                     (src/activation_cuda.cu:510-544)        -> tagi_relu_fwd
//   BaseLayerCuda::update_weights / update_biases (src/base_layer_cuda.cu:161-202) -> tagi_param_update
//   HiddenStateCuda::set_input_x          (src/data_struct_cuda.cu:39-63)         -> one copy of the batch, fills on the device
// Everything else of those classes (constructors, parameter storage, save / load, to_host, bindings) stays cuTAGI's own
// code: its translation units are compiled unchanged and only the symbols of the methods above are weakened in the
// resulting objects (objcopy --weaken-symbol, integration/Makefile), so that the definitions here win at link time.
//
// Behaviour follows cuTAGI's CPU classes, which are the reference for parity: BatchNorm2d uses the unbiased variance
// (divisor n - 1) and replaces the running averages on the first training batch (src/batchnorm_layer.cpp:127-168,
// 862-868); cuTAGI's CUDA class divides by n and has that rule commented out (src/batchnorm_layer_cuda.cu:857-862,
// 931-940). Pooling needs no index tables here; the class still builds its own once (its destructor frees them).
#include "activation_cuda.cuh"
#include "base_layer_cuda.cuh"
#include "batchnorm_layer_cuda.cuh"
#include "custom_logger.h"
#include "data_struct_cuda.cuh"
#include "ddp_b200_hooks.h"
#include "pooling_layer_cuda.cuh"
#include "tagi_b200.h"

#include <cstring>
#include <thread>
#include <vector>

namespace {
void require_ok(int status) {
    if (status != TAGI_OK) LOG(LogLevel::ERROR, std::string("tagi_b200: ") + tagi_last_error_string());
}
// the batch size whose cap factor (src/base_layer.cpp:164-187: 0.1, 2, 3) equals the layer's current one
int batch_for_cap(float cap) { return cap < 1.0f ? 1 : cap < 2.5f ? 2 : 256; }
}  // namespace

// ------------------------------------------------------------------------------------------------ BatchNorm2d
void BatchNorm2dCuda::forward(BaseHiddenStates &input_states, BaseHiddenStates &output_states, BaseTempStates &) {
    auto *in = dynamic_cast<HiddenStateCuda *>(&input_states);
    auto *out = dynamic_cast<HiddenStateCuda *>(&output_states);
    const int batch = static_cast<int>(input_states.block_size);
    set_cap_factor_udapte(batch);
    if (input_size == 0 || output_size == 0) {
        input_size = input_states.actual_size;
        output_size = input_states.actual_size;
    }
    float m = momentum;
    if (first_batch) {   // the CPU class's rule: the first training batch replaces the running averages
        if (training) m = 0.0f;
        first_batch = false;
    }
    output_states.width = out_width;
    output_states.height = out_height;
    output_states.depth = out_channels;
    output_states.block_size = batch;
    output_states.actual_size = output_size;
    // per-channel statistics over (batch, pixels); a layer used on plain feature vectors is the same with one pixel
    const bool spatial = num_features == static_cast<int>(in_channels);
    const int channels = spatial ? static_cast<int>(in_channels) : static_cast<int>(input_size);
    const int wihi = spatial ? static_cast<int>(in_height * in_width) : 1;
    require_ok(tagi_bn2d_fwd(batch, channels, wihi, bias ? 1 : 0, training ? 1 : 0, epsilon, m, d_mu_w, d_var_w, d_mu_b,
                             d_var_b, in->d_mu_a, in->d_var_a, d_mu_ra, d_var_ra, d_mu_norm_batch, d_var_norm_batch,
                             out->d_mu_a, out->d_var_a, nullptr));
    if (training) store_states_for_training_cuda(*in, *out);
}

void BatchNorm2dCuda::backward(BaseDeltaStates &input_delta_states, BaseDeltaStates &output_delta_states,
                               BaseTempStates &, bool state_udapte) {
    auto *saved = dynamic_cast<BackwardStateCuda *>(bwd_states.get());
    auto *din = dynamic_cast<DeltaStateCuda *>(&input_delta_states);
    auto *dout = dynamic_cast<DeltaStateCuda *>(&output_delta_states);
    const int batch = static_cast<int>(input_delta_states.block_size);
    const bool spatial = in_channels != 0;
    const int channels = spatial ? static_cast<int>(in_channels) : static_cast<int>(input_size);
    const int wihi = spatial ? static_cast<int>(in_height * in_width) : 1;
    if (!param_update && !state_udapte) return;
    // one pass produces the state deltas and all four parameter deltas
    require_ok(tagi_bn2d_bwd(batch, channels, wihi, bias ? 1 : 0, state_udapte ? 1 : 0, epsilon, d_mu_w, d_var_w, d_var_b,
                             saved->d_mu_a, saved->d_jcb, d_mu_norm_batch, d_var_norm_batch, din->d_delta_mu,
                             din->d_delta_var, dout->d_delta_mu, dout->d_delta_var, d_delta_mu_w, d_delta_var_w,
                             d_delta_mu_b, d_delta_var_b, nullptr));
    if (param_update) {
        ddp_b200_deltas_ready(d_delta_mu_w);
        ddp_b200_deltas_ready(d_delta_var_w);
        if (bias) {
            ddp_b200_deltas_ready(d_delta_mu_b);
            ddp_b200_deltas_ready(d_delta_var_b);
        }
    }
}

// ------------------------------------------------------------------------------------------------ AvgPool2d
namespace {
tagi_conv2d_geom pool_geometry(const AvgPool2dCuda &l, int batch) {
    tagi_conv2d_geom g;
    g.B = batch;
    g.fi = g.fo = static_cast<int>(l.in_channels);
    g.hi = static_cast<int>(l.in_height), g.wi = static_cast<int>(l.in_width);
    g.ho = static_cast<int>(l.out_height), g.wo = static_cast<int>(l.out_width);
    g.k = static_cast<int>(l.kernel_size);
    g.stride = l.stride > 0 ? l.stride : g.k;   // global pooling is written as stride -1
    g.pad = l.padding, g.pad_type = l.padding_type, g.has_bias = 0;
    return g;
}
}  // namespace

void AvgPool2dCuda::forward(BaseHiddenStates &input_states, BaseHiddenStates &output_states, BaseTempStates &) {
    auto *in = dynamic_cast<HiddenStateCuda *>(&input_states);
    auto *out = dynamic_cast<HiddenStateCuda *>(&output_states);
    const int batch = static_cast<int>(input_states.block_size);
    // cuTAGI's class owns two device index tables that its destructor frees; they are built once here as the original
    // does on its first forward pass, so that every other method of the class finds the object as it expects it. The
    // kernels below do not read them.
    if (pool_idx.size() == 0) lazy_index_init();
    out->width = out_width;
    out->height = out_height;
    out->depth = out_channels;
    out->block_size = batch;
    out->actual_size = output_size;
    const tagi_conv2d_geom g = pool_geometry(*this, batch);
    require_ok(tagi_avgpool2d_fwd(&g, in->d_mu_a, in->d_var_a, out->d_mu_a, out->d_var_a, nullptr));
    if (training) store_states_for_training_cuda(*in, *out);
}

void AvgPool2dCuda::backward(BaseDeltaStates &input_delta_states, BaseDeltaStates &output_delta_states, BaseTempStates &,
                             bool state_udapte) {
    if (!state_udapte) return;
    auto *saved = dynamic_cast<BackwardStateCuda *>(bwd_states.get());
    auto *din = dynamic_cast<DeltaStateCuda *>(&input_delta_states);
    auto *dout = dynamic_cast<DeltaStateCuda *>(&output_delta_states);
    const tagi_conv2d_geom g = pool_geometry(*this, static_cast<int>(input_delta_states.block_size));
    require_ok(tagi_avgpool2d_bwd_state(&g, saved->d_jcb, din->d_delta_mu, din->d_delta_var, dout->d_delta_mu,
                                        dout->d_delta_var, nullptr));
}

// ------------------------------------------------------------------------------------------------ ReLU
void ReLUCuda::forward(BaseHiddenStates &input_states, BaseHiddenStates &output_states, BaseTempStates &) {
    auto *in = dynamic_cast<HiddenStateCuda *>(&input_states);
    auto *out = dynamic_cast<HiddenStateCuda *>(&output_states);
    out->width = in->width;
    out->height = in->height;
    out->depth = in->depth;
    out->block_size = in->block_size;
    out->actual_size = in->actual_size;
    const size_t n = static_cast<size_t>(input_states.actual_size) * input_states.block_size;
    require_ok(tagi_relu_fwd(in->d_mu_a, in->d_var_a, n, out->d_mu_a, out->d_var_a, out->d_jcb, nullptr));
    if (input_size != input_states.actual_size) {
        input_size = input_states.actual_size;
        output_size = input_states.actual_size;
    }
}

// ------------------------------------------------------------------------------------------------ capped update
void BaseLayerCuda::update_weights() {
    neg_var_w_counter = 0;
    if (num_weights == 0 || d_mu_w == nullptr || d_neg_var_count == nullptr) return;   // a layer without parameters
    // the counter of negative variances is reset and counted on the device; one read-back keeps the host member current
    if (cudaMemsetAsync(d_neg_var_count, 0, sizeof(int), nullptr) != cudaSuccess)
        LOG(LogLevel::ERROR, "Failed to reset the negative-variance counter");
    require_ok(tagi_param_update(batch_for_cap(cap_factor_update), num_weights, d_mu_w, d_var_w, d_delta_mu_w, d_delta_var_w,
                                 d_neg_var_count, nullptr));
    if (cudaMemcpy(&neg_var_w_counter, d_neg_var_count, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
        LOG(LogLevel::ERROR, "Failed to copy negative var count from device");
}

void BaseLayerCuda::update_biases() {
    if (!bias || num_biases == 0 || d_mu_b == nullptr) return;
    require_ok(tagi_param_update(batch_for_cap(cap_factor_update), num_biases, d_mu_b, d_var_b, d_delta_mu_b, d_delta_var_b,
                                 nullptr, nullptr));
}

// ------------------------------------------------------------------------------------------------ network input
// cuTAGI copies the batch element by element into the state's host vectors (means, a variance of zero or the given one,
// Jacobians of one) and then uploads all three from pageable memory. Here the means go to the device in one copy straight
// from the caller's vector and the other two arrays are written on the device; for the 64 x 3 x 224 x 224 batch of the
// ResNet-18 configuration that is one 38.5 MB copy instead of three plus 29 million host-side assignments. The host
// mirrors keep whatever they held: cuTAGI reads them only after to_host(), which overwrites them.
namespace {
__global__ void fill_input_aux_kernel(size_t n, bool zero_var, float *var_a, float *jcb) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        if (zero_var) var_a[i] = 0.0f;
        jcb[i] = 1.0f;
    }
}
}  // namespace

namespace {
// Large batches go through a pinned staging buffer that a few host threads fill, followed by one asynchronous copy on
// the legacy stream: the copy out of pageable memory that cudaMemcpy would do by itself ran at about 5 GB/s on the
// benchmark host (38.5 MB in 8 ms), four threads fill the staging buffer at several times that, and the call returns
// while the DMA is still running. One staging buffer per process: cuTAGI drives a model from one host thread.
struct InputStaging {
    float *pinned = nullptr;
    size_t capacity = 0;       // floats
    cudaEvent_t drained = nullptr;   // the last copy out of the buffer has finished
};
InputStaging g_staging;

void threaded_copy(float *dst, const float *src, size_t n) {
    const unsigned hw = std::thread::hardware_concurrency();
    const size_t nt = hw >= 8 ? 4 : hw >= 4 ? 2 : 1;
    if (nt == 1) {
        std::memcpy(dst, src, n * sizeof(float));
        return;
    }
    std::vector<std::thread> workers;
    const size_t per = (n + nt - 1) / nt;
    for (size_t t = 0; t < nt; t++) {
        const size_t b = t * per, e = b + per < n ? b + per : n;
        if (b >= e) break;
        workers.emplace_back([=] { std::memcpy(dst + b, src + b, (e - b) * sizeof(float)); });
    }
    for (auto &w : workers) w.join();
}

// true when the batch was handed to the staged path
bool staged_upload(float *device_dst, const float *src, size_t n) {
    if (n * sizeof(float) < (1u << 20)) return false;   // small batches: the plain copy is as fast
    InputStaging &st = g_staging;
    if (st.drained == nullptr && cudaEventCreateWithFlags(&st.drained, cudaEventDisableTiming) != cudaSuccess) return false;
    if (st.capacity < n) {
        if (st.pinned != nullptr) {
            cudaEventSynchronize(st.drained);
            cudaFreeHost(st.pinned);
            st.pinned = nullptr, st.capacity = 0;
        }
        if (cudaHostAlloc(reinterpret_cast<void **>(&st.pinned), n * sizeof(float), cudaHostAllocDefault) != cudaSuccess) {
            cudaGetLastError();   // no pinned memory to be had: the caller copies directly
            st.pinned = nullptr;
            return false;
        }
        st.capacity = n;
    } else {
        cudaEventSynchronize(st.drained);   // the previous batch has left the buffer (long ago, normally)
    }
    threaded_copy(st.pinned, src, n);
    if (cudaMemcpyAsync(device_dst, st.pinned, n * sizeof(float), cudaMemcpyHostToDevice, nullptr) != cudaSuccess) return false;
    cudaEventRecord(st.drained, nullptr);
    return true;
}
}  // namespace

void tagi_b200_upload_input(HiddenStateCuda &state, const float *mu, const float *var, size_t n, size_t block_size) {
    state.actual_size = n / block_size;
    state.block_size = block_size;
    if (n > state.size) LOG(LogLevel::ERROR, "Input batch is larger than the hidden-state buffer");
    cudaSetDevice(state.device_idx);
    cudaError_t e = cudaSuccess;
    if (!staged_upload(state.d_mu_a, mu, n)) e = cudaMemcpy(state.d_mu_a, mu, n * sizeof(float), cudaMemcpyHostToDevice);
    if (e == cudaSuccess && var != nullptr) e = cudaMemcpy(state.d_var_a, var, n * sizeof(float), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) LOG(LogLevel::ERROR, std::string("Failed to copy the input batch to the device: ") + cudaGetErrorString(e));
    if (n > 0) {
        const unsigned blocks = (unsigned)((n + 1023) / 1024 < 148 * 8 ? (n + 1023) / 1024 : 148 * 8);
        fill_input_aux_kernel<<<blocks, 256>>>(n, var == nullptr, state.d_var_a, state.d_jcb);
        if (cudaGetLastError() != cudaSuccess) LOG(LogLevel::ERROR, "Failed to launch the input fill kernel");
    }
}

void HiddenStateCuda::set_input_x(const std::vector<float> &mu_x, const std::vector<float> &var_x, const size_t block_size) {
    const size_t n = mu_x.size();
    tagi_b200_upload_input(*this, mu_x.data(), var_x.size() == n ? var_x.data() : nullptr, n, block_size);
}
