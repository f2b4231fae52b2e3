// Host I/O of cuTAGI's Sequential for the drop-in build: the two methods pytagi calls once per training step.
//   Sequential::forward_py   (src/sequential.cpp:771-789)  numpy batch in
//   Sequential::get_outputs  (src/sequential.cpp:791-814)  predictions out
// cuTAGI's own bodies copy the numpy batch into a fresh std::vector, then element by element into the hidden state's
// host vectors, then upload three arrays from pageable memory; on the way out they download the whole ping-pong buffer
// (three arrays of batch x widest layer: 616 MB for the ResNet-18 configuration) to read batch x 11 numbers. Here the
// batch goes from the numpy buffer to the device in one copy (variance and Jacobian are written on the device), and the
// read-back moves exactly batch x n_out means and variances. Measured on the ResNet-18 configuration: the forward call
// spent 21.6 ms on the host before its first kernel, and get_outputs 60 ms in the download.
// Everything else of Sequential is cuTAGI's code: the two symbols are weakened in its object (integration/Makefile).
// On the CPU device both methods behave as cuTAGI's do.
#include <cuda_runtime.h>

#include "custom_logger.h"
#include "data_struct_cuda.cuh"
#include "ddp_b200_hooks.h"
#include "sequential.h"

// neighbours_b200.cu: one upload of the batch's means (and variances when given), variance / Jacobian fill on the device
void tagi_b200_upload_input(HiddenStateCuda &state, const float *mu, const float *var, size_t n, size_t block_size);

void Sequential::forward_py(pybind11::array_t<float> mu_a_np, pybind11::array_t<float> var_a_np) {
    auto mu_buf = mu_a_np.request();
    const float *mu_ptr = static_cast<const float *>(mu_buf.ptr);
    const size_t n = static_cast<size_t>(mu_buf.size);
    const float *var_ptr = nullptr;
    size_t n_var = 0;
    pybind11::buffer_info var_buf;
    if (!var_a_np.is_none()) {
        var_buf = var_a_np.request();
        var_ptr = static_cast<const float *>(var_buf.ptr);
        n_var = static_cast<size_t>(var_buf.size);
    }
    if (this->device.compare("cuda") != 0) {   // CPU model: cuTAGI's own path
        std::vector<float> mu_a(mu_ptr, mu_ptr + n);
        if (var_ptr) {
            std::vector<float> var_a(var_ptr, var_ptr + n_var);
            this->forward(mu_a, var_a);
        } else {
            this->forward(mu_a);
        }
        return;
    }
    // batch size and buffers, as Sequential::forward(mu_x, var_x) sets them up (src/sequential.cpp:279-318)
    const int in_size = this->layers.front()->get_input_size();
    if (in_size <= 0 || n % in_size != 0)
        LOG(LogLevel::ERROR, "Input size mismatch: " + std::to_string(in_size) + " vs " + std::to_string(n));
    const int batch = static_cast<int>(n / in_size);
    if (this->z_buffer_block_size == 0) {   // first batch: the buffers are sized for it
        this->z_buffer_block_size = batch;
        this->z_buffer_size = batch * this->z_buffer_size;
        this->init_output_state_buffer();
        if (this->training) this->init_delta_state_buffer();
    }
    if (batch != this->z_buffer_block_size) {   // another batch size: same per-sample width, new capacity
        this->z_buffer_size = batch * (this->z_buffer_size / this->z_buffer_block_size);
        this->z_buffer_block_size = batch;
        this->input_z_buffer->set_size(this->z_buffer_size, batch);
        if (this->training) {
            this->input_delta_z_buffer->set_size(this->z_buffer_size, batch);
            this->output_delta_z_buffer->set_size(this->z_buffer_size, batch);
        }
    }
    auto *in = dynamic_cast<HiddenStateCuda *>(this->input_z_buffer.get());
    if (in == nullptr) LOG(LogLevel::ERROR, "The input buffer of a CUDA model is not a HiddenStateCuda");
    tagi_b200_upload_input(*in, mu_ptr, n_var == n ? var_ptr : nullptr, n, static_cast<size_t>(batch));

    for (auto &layer : this->layers) {
        layer->forward(*this->input_z_buffer, *this->output_z_buffer, *this->temp_states);
        std::swap(this->input_z_buffer, this->output_z_buffer);
    }
    std::swap(this->output_z_buffer, this->input_z_buffer);   // the last layer's output is the network's
}

std::tuple<pybind11::array_t<float>, pybind11::array_t<float>> Sequential::get_outputs() {
    const int batch = static_cast<int>(this->output_z_buffer->block_size);
    const int n_out = static_cast<int>(this->layers.back()->output_size);
    const size_t n = static_cast<size_t>(batch) * n_out;
    pybind11::array_t<float> mu(n), var(n);
    float *mu_out = mu.mutable_data(), *var_out = var.mutable_data();
    auto *out = this->device.compare("cuda") == 0 ? dynamic_cast<HiddenStateCuda *>(this->output_z_buffer.get()) : nullptr;
    if (out != nullptr) {
        // exactly batch x n_out moments; a blocking copy on the legacy stream, i.e. after every kernel of the step
        cudaSetDevice(out->device_idx);
        cudaError_t e = cudaMemcpy(mu_out, out->d_mu_a, n * sizeof(float), cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) e = cudaMemcpy(var_out, out->d_var_a, n * sizeof(float), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess)
            LOG(LogLevel::ERROR, std::string("Failed to read the network outputs back: ") + cudaGetErrorString(e));
        tagi_b200_raise_on_kernel_abort();   // the device is idle here: the place to notice an aborted tensor-core kernel
        // the state's host mirror keeps what cuTAGI would have left in these entries
        for (size_t j = 0; j < n && j < out->mu_a.size(); j++) out->mu_a[j] = mu_out[j], out->var_a[j] = var_out[j];
    } else {
        for (size_t j = 0; j < n; j++) mu_out[j] = this->output_z_buffer->mu_a[j], var_out[j] = this->output_z_buffer->var_a[j];
    }
    return {mu, var};
}
