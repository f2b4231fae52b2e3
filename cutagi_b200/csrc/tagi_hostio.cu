// Host I/O path of a training step (include/tagi_b200.h, "tagi_io_*"): pinned, multi-slot staging of a batch's inputs,
// observations and selected indices, asynchronous upload on a stream of its own, and a read-back of exactly the
// B x n_out output moments. cuTAGI copies a whole state buffer (capacity = batch x widest layer) in both directions with
// blocking cudaMemcpy from pageable vectors (HiddenStateCuda::to_device / to_host, src/data_struct_cuda.cu:83-123;
// ObservationCuda::to_device, :300-330) and its Python layer turns the observations into lists first
// (pytagi/nn/output_updater.py:45-47); for the small configurations those copies, not the kernels, are the step.
#include <new>

#include "tagi_common.h"

struct tagi_io {
    int depth = 0, device = 0;
    size_t in_floats = 0, obs_floats = 0, idx_ints = 0, out_floats = 0;
    // per slot: one pinned block and one device block laid out [inputs | observations | indices], pinned outputs [mu | var]
    char **h_in = nullptr, **d_in = nullptr;
    float **h_out = nullptr;
    cudaEvent_t *uploaded = nullptr, *consumed = nullptr, *downloaded = nullptr;
    bool *has_consumed = nullptr;
    cudaStream_t up = nullptr, down = nullptr;
    cudaEvent_t ready = nullptr;
    size_t block_bytes() const { return (in_floats + obs_floats) * sizeof(float) + idx_ints * sizeof(int); }
};

using namespace tagi;

namespace {
int bad_slot(const tagi_io *io, int slot, const char *who) {
    if (!io) return fail(TAGI_ERR_INVALID_ARGUMENT, std::string(who) + ": null pipeline");
    if (slot < 0 || slot >= io->depth) return fail(TAGI_ERR_INVALID_ARGUMENT, std::string(who) + ": slot out of range");
    return TAGI_OK;
}
}  // namespace

extern "C" {

int tagi_io_create(size_t in_floats, size_t obs_floats, size_t idx_ints, size_t out_floats, int depth, tagi_io **out) {
    TAGI_REQUIRE(out != nullptr, "null output pointer");
    TAGI_REQUIRE(depth >= 1 && depth <= 8, "depth must be 1 .. 8");
    TAGI_REQUIRE(in_floats > 0 && out_floats > 0, "input and output sizes must be positive");
    tagi_io *io = new (std::nothrow) tagi_io;
    if (!io) return fail(TAGI_ERR_CUDA, "out of host memory");
    io->depth = depth, io->in_floats = in_floats, io->obs_floats = obs_floats, io->idx_ints = idx_ints, io->out_floats = out_floats;
    cudaError_t e = cudaGetDevice(&io->device);
    io->h_in = new char *[depth](), io->d_in = new char *[depth](), io->h_out = new float *[depth]();
    io->uploaded = new cudaEvent_t[depth](), io->consumed = new cudaEvent_t[depth](), io->downloaded = new cudaEvent_t[depth]();
    io->has_consumed = new bool[depth]();
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&io->up, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&io->down, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&io->ready, cudaEventDisableTiming);
    for (int s = 0; s < depth && e == cudaSuccess; s++) {
        e = cudaHostAlloc(reinterpret_cast<void **>(&io->h_in[s]), io->block_bytes(), cudaHostAllocDefault);
        if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&io->d_in[s]), io->block_bytes());
        if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void **>(&io->h_out[s]), 2 * out_floats * sizeof(float), cudaHostAllocDefault);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&io->uploaded[s], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&io->consumed[s], cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&io->downloaded[s], cudaEventDisableTiming);
    }
    if (e != cudaSuccess) {
        const int rc = cuda_fail(e, "tagi_io_create");
        const std::string msg = last_error();
        tagi_io_destroy(io);
        last_error() = msg;
        return rc;
    }
    *out = io;
    return TAGI_OK;
}

int tagi_io_destroy(tagi_io *io) {
    if (!io) return TAGI_OK;
    if (io->up) cudaStreamSynchronize(io->up);
    if (io->down) cudaStreamSynchronize(io->down);
    for (int s = 0; s < io->depth; s++) {
        if (io->h_in && io->h_in[s]) cudaFreeHost(io->h_in[s]);
        if (io->d_in && io->d_in[s]) cudaFree(io->d_in[s]);
        if (io->h_out && io->h_out[s]) cudaFreeHost(io->h_out[s]);
        if (io->uploaded && io->uploaded[s]) cudaEventDestroy(io->uploaded[s]);
        if (io->consumed && io->consumed[s]) cudaEventDestroy(io->consumed[s]);
        if (io->downloaded && io->downloaded[s]) cudaEventDestroy(io->downloaded[s]);
    }
    if (io->ready) cudaEventDestroy(io->ready);
    if (io->up) cudaStreamDestroy(io->up);
    if (io->down) cudaStreamDestroy(io->down);
    delete[] io->h_in;
    delete[] io->d_in;
    delete[] io->h_out;
    delete[] io->uploaded;
    delete[] io->consumed;
    delete[] io->downloaded;
    delete[] io->has_consumed;
    delete io;
    return TAGI_OK;
}

int tagi_io_host_buffers(tagi_io *io, int slot, float **inputs, float **obs, int **idx) {
    int rc = bad_slot(io, slot, __func__);
    if (rc != TAGI_OK) return rc;
    if (inputs) *inputs = reinterpret_cast<float *>(io->h_in[slot]);
    if (obs) *obs = reinterpret_cast<float *>(io->h_in[slot]) + io->in_floats;
    if (idx) *idx = reinterpret_cast<int *>(reinterpret_cast<float *>(io->h_in[slot]) + io->in_floats + io->obs_floats);
    return TAGI_OK;
}

int tagi_io_device_buffers(tagi_io *io, int slot, const float **inputs, const float **obs, const int **idx) {
    int rc = bad_slot(io, slot, __func__);
    if (rc != TAGI_OK) return rc;
    if (inputs) *inputs = reinterpret_cast<const float *>(io->d_in[slot]);
    if (obs) *obs = reinterpret_cast<const float *>(io->d_in[slot]) + io->in_floats;
    if (idx) *idx = reinterpret_cast<const int *>(reinterpret_cast<const float *>(io->d_in[slot]) + io->in_floats + io->obs_floats);
    return TAGI_OK;
}

int tagi_io_upload(tagi_io *io, int slot, void *compute_stream) {
    int rc = bad_slot(io, slot, __func__);
    if (rc != TAGI_OK) return rc;
    // the step that last read this slot's device buffers must have finished with them
    if (io->has_consumed[slot]) TAGI_CUDA(cudaStreamWaitEvent(io->up, io->consumed[slot], 0));
    TAGI_CUDA(cudaMemcpyAsync(io->d_in[slot], io->h_in[slot], io->block_bytes(), cudaMemcpyHostToDevice, io->up));
    TAGI_CUDA(cudaEventRecord(io->uploaded[slot], io->up));
    TAGI_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(compute_stream), io->uploaded[slot], 0));
    return TAGI_OK;
}

int tagi_io_consumed(tagi_io *io, int slot, void *compute_stream) {
    int rc = bad_slot(io, slot, __func__);
    if (rc != TAGI_OK) return rc;
    TAGI_CUDA(cudaEventRecord(io->consumed[slot], static_cast<cudaStream_t>(compute_stream)));
    io->has_consumed[slot] = true;
    return TAGI_OK;
}

int tagi_io_download(tagi_io *io, int slot, const float *mu, const float *var, size_t n, void *compute_stream) {
    int rc = bad_slot(io, slot, __func__);
    if (rc != TAGI_OK) return rc;
    TAGI_REQUIRE(mu != nullptr && var != nullptr, "null output moments");
    TAGI_REQUIRE(n > 0 && n <= io->out_floats, "n exceeds the pipeline's output capacity");
    TAGI_CUDA(cudaEventRecord(io->ready, static_cast<cudaStream_t>(compute_stream)));
    TAGI_CUDA(cudaStreamWaitEvent(io->down, io->ready, 0));
    TAGI_CUDA(cudaMemcpyAsync(io->h_out[slot], mu, n * sizeof(float), cudaMemcpyDeviceToHost, io->down));
    TAGI_CUDA(cudaMemcpyAsync(io->h_out[slot] + io->out_floats, var, n * sizeof(float), cudaMemcpyDeviceToHost, io->down));
    TAGI_CUDA(cudaEventRecord(io->downloaded[slot], io->down));
    return TAGI_OK;
}

int tagi_io_wait_output(tagi_io *io, int slot, const float **mu, const float **var) {
    int rc = bad_slot(io, slot, __func__);
    if (rc != TAGI_OK) return rc;
    TAGI_CUDA(cudaEventSynchronize(io->downloaded[slot]));
    if (mu) *mu = io->h_out[slot];
    if (var) *var = io->h_out[slot] + io->out_floats;
    return TAGI_OK;
}

}  // extern "C"
