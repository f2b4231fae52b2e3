// Drop-in implementation of cuTAGI's data-parallel classes (declared in include/ddp.h:26-145 of the cuTAGI tree) on
// top of libtagi_b200_comm's C ABI, linked into the cuTAGI module in place of src/ddp.cpp:
//   DDPConfig       constructor                                                   (src/ddp.cpp:17-23)
//   Communicator    a subclass over tagi_comm_* replaces NCCLCommunicator          (src/ddp.cpp:27-72)
//   DDPSequential   constructor, sync_parameters, sync_base_parameters, step, ... (src/ddp.cpp:76-193)
// Differences from the original, on purpose:
//   * no MPI: the NCCL id travels through a rendezvous file (TAGI_B200_RENDEZVOUS, else a path derived from
//     MASTER_ADDR / MASTER_PORT), so `torchrun` or any launcher that sets RANK / WORLD_SIZE works;
//   * parameter tensors are enumerated through LayerBlock and ResNetBlock containers (the original walks the top-level
//     layer list only and never exchanges anything inside a residual block);
//   * parameters are broadcast after preinit_layer(), i.e. after the Conv2d layers have created theirs (the original
//     broadcasts before the first forward pass, when they do not exist yet);
//   * the deltas are registered once, in backward order, and packed into buckets; LinearCuda / Conv2dCuda announce their
//     deltas from inside backward() (ddp_b200_hooks.h), so a bucket's allreduce overlaps the rest of the backward pass;
//     step() launches what is left and makes the default stream wait before the update.
#include "ddp.h"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <unistd.h>

#include <cstdlib>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "base_layer_cuda.cuh"
#include "custom_logger.h"
#include "ddp_b200_hooks.h"
#include "ddp_b200_walk.h"
#include "layer_block.h"
#include "resnet_block.h"
#include "resnet_block_cuda.cuh"
#include "tagi_b200.h"
#include "tagi_b200_comm.h"

namespace {

// libtagi_b200_comm.so (and through it NCCL) is loaded when the first DDPSequential is built, not when the module is
// imported: single-GPU users never touch NCCL, and a process that also holds another copy of NCCL (PyTorch ships one)
// binds to whichever is resident by then. TAGI_B200_COMM_LIB overrides the path (default: next to libtagi_b200.so).
struct CommApi {
#define TAGI_COMM_FN(name) decltype(&::name) name = nullptr;
    TAGI_COMM_FN(tagi_comm_last_error_string)
    TAGI_COMM_FN(tagi_comm_init_file)
    TAGI_COMM_FN(tagi_comm_register)
    TAGI_COMM_FN(tagi_comm_finalize_buckets)
    TAGI_COMM_FN(tagi_comm_tensor_ready)
    TAGI_COMM_FN(tagi_comm_flush)
    TAGI_COMM_FN(tagi_comm_wait)
    TAGI_COMM_FN(tagi_comm_allreduce)
    TAGI_COMM_FN(tagi_comm_broadcast)
    TAGI_COMM_FN(tagi_comm_check)
    TAGI_COMM_FN(tagi_comm_sync_stream)
    TAGI_COMM_FN(tagi_comm_barrier)
    TAGI_COMM_FN(tagi_comm_destroy)
#undef TAGI_COMM_FN
};
CommApi &comm() {
    static CommApi api = [] {
        CommApi a;
        std::string path;
        if (const char *p = std::getenv("TAGI_B200_COMM_LIB")) {
            path = p;
        } else {
            Dl_info info;
            // libtagi_b200.so's directory: tagi_version lives there
            if (dladdr(reinterpret_cast<void *>(&tagi_version), &info) && info.dli_fname) {
                path = info.dli_fname;
                path = path.substr(0, path.find_last_of('/') + 1) + "libtagi_b200_comm.so";
            } else {
                path = "libtagi_b200_comm.so";
            }
        }
        void *h = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
        if (!h) LOG(LogLevel::ERROR, std::string("cannot load ") + path + ": " + dlerror());
#define TAGI_COMM_FN(name)                                                         \
    a.name = reinterpret_cast<decltype(a.name)>(dlsym(h, #name));                  \
    if (!a.name) LOG(LogLevel::ERROR, std::string("missing symbol " #name " in ") + path);
        TAGI_COMM_FN(tagi_comm_last_error_string)
        TAGI_COMM_FN(tagi_comm_init_file)
        TAGI_COMM_FN(tagi_comm_register)
        TAGI_COMM_FN(tagi_comm_finalize_buckets)
        TAGI_COMM_FN(tagi_comm_tensor_ready)
        TAGI_COMM_FN(tagi_comm_flush)
        TAGI_COMM_FN(tagi_comm_wait)
        TAGI_COMM_FN(tagi_comm_allreduce)
        TAGI_COMM_FN(tagi_comm_broadcast)
        TAGI_COMM_FN(tagi_comm_check)
        TAGI_COMM_FN(tagi_comm_sync_stream)
        TAGI_COMM_FN(tagi_comm_barrier)
        TAGI_COMM_FN(tagi_comm_destroy)
#undef TAGI_COMM_FN
        return a;
    }();
    return api;
}

void require_ok(int status, const char *what) {
    if (status != TAGI_OK) LOG(LogLevel::ERROR, std::string(what) + ": " + comm().tagi_comm_last_error_string());
}

// ResNetBlockCuda keeps its two sub-blocks private and has no accessor. Explicit template instantiation may name
// private members, which gives a pointer-to-member without touching cuTAGI's header.
template <class Tag, typename Tag::type Member>
struct Expose {
    friend typename Tag::type reach(Tag) { return Member; }
};
struct MainBlockTag {
    typedef std::shared_ptr<BaseLayer> ResNetBlockCuda::*type;
    friend type reach(MainBlockTag);
};
struct ShortcutTag {
    typedef std::shared_ptr<BaseLayer> ResNetBlockCuda::*type;
    friend type reach(ShortcutTag);
};
template struct Expose<MainBlockTag, &ResNetBlockCuda::main_block>;
template struct Expose<ShortcutTag, &ResNetBlockCuda::shortcut>;

// children of a container in forward order; 0 = leaf, 1 = sequence, 2 = residual block (main block, shortcut)
int children_of(BaseLayer *layer, std::vector<BaseLayer *> &out) {
    if (auto *blk = dynamic_cast<LayerBlock *>(layer)) {
        for (auto &l : blk->layers) out.push_back(l.get());
        return 1;
    }
    if (auto *res = dynamic_cast<ResNetBlockCuda *>(layer)) {
        out.push_back((res->*reach(MainBlockTag())).get());
        if (auto s = (res->*reach(ShortcutTag())).get()) out.push_back(s);
        return 2;
    }
    if (auto *res = dynamic_cast<ResNetBlock *>(layer)) {
        out.push_back(res->main_block.get());
        if (res->shortcut) out.push_back(res->shortcut.get());
        return 2;
    }
    return 0;
}

// Every CUDA layer that owns parameters, in the order the backward pass finishes them
std::vector<BaseLayerCuda *> parameter_layers_backward(Sequential &model) {
    std::vector<BaseLayer *> top;
    for (auto &l : model.layers) top.push_back(l.get());
    std::vector<BaseLayerCuda *> out;
    ddp_b200_walk_backward(top, children_of, [&](BaseLayer *l) {
        auto type = l->get_layer_type();
        if (type == LayerType::Activation || type == LayerType::Pool2d) return;
        auto *cu = dynamic_cast<BaseLayerCuda *>(l);
        if (!cu) {
            LOG(LogLevel::ERROR, "Layer is not a CUDA layer: " + l->get_layer_info());
            return;
        }
        if (cu->num_weights > 0) out.push_back(cu);
    });
    return out;
}

// tensor index in the exchange by device address (filled by DDPSequential's constructor)
std::unordered_map<const float *, int> g_registered;
bool g_average = true;

class B200Communicator : public Communicator {
    int rank_, world_;

   public:
    B200Communicator(int rank, int world, int device, const std::string &path) : rank_(rank), world_(world) {
        const char *t = std::getenv("TAGI_B200_RENDEZVOUS_TIMEOUT_MS");
        require_ok(comm().tagi_comm_init_file(path.c_str(), rank, world, device, t ? std::atoi(t) : 120000), "tagi_comm_init_file");
    }
    ~B200Communicator() override {
        g_registered.clear();
        comm().tagi_comm_destroy();
    }
    // blocking, as NCCLCommunicator's (src/ddp.cpp:53-57): the collective runs on the exchange's stream, ordered after
    // the legacy default stream, and the host waits for it
    void all_reduce(float *data, size_t count, bool average = false) override {
        require_ok(comm().tagi_comm_allreduce(data, count, average ? 1 : 0, nullptr), "tagi_comm_allreduce");
        require_ok(comm().tagi_comm_sync_stream(), "tagi_comm_sync_stream");
    }
    void broadcast(float *data, size_t count, int root) override {
        require_ok(comm().tagi_comm_broadcast(data, count, root, nullptr), "tagi_comm_broadcast");
        require_ok(comm().tagi_comm_sync_stream(), "tagi_comm_sync_stream");
    }
    void barrier() override { require_ok(comm().tagi_comm_barrier(), "tagi_comm_barrier"); }
    int get_rank() const override { return rank_; }
    int get_world_size() const override { return world_; }
    void check_async_error() override { require_ok(comm().tagi_comm_check(), "tagi_comm_check"); }
};

std::string rendezvous_path() {
    if (const char *p = std::getenv("TAGI_B200_RENDEZVOUS")) return p;
    const char *addr = std::getenv("MASTER_ADDR"), *port = std::getenv("MASTER_PORT");
    std::string s = "/tmp/tagi_b200_ddp_" + std::to_string((long)getuid());
    if (addr) s += std::string("_") + addr;
    if (port) s += std::string("_") + port;
    return s;
}

}  // namespace

void ddp_b200_deltas_ready(const float *device_ptr) {
    if (g_registered.empty()) return;
    auto it = g_registered.find(device_ptr);
    if (it == g_registered.end()) return;
    require_ok(comm().tagi_comm_tensor_ready(it->second, nullptr, g_average ? 1 : 0), "tagi_comm_tensor_ready");
}

void tagi_b200_raise_on_kernel_abort() {
    int status = 0;
    if (tagi_tc_status(&status, 1) != TAGI_OK)
        LOG(LogLevel::ERROR, std::string("tagi_b200: ") + tagi_last_error_string());
    if (status != 0)
        LOG(LogLevel::ERROR, "tagi_b200: a bounded device-side wait of the tensor-core kernels ran out (status " +
                                 std::to_string(status) + "); outputs of that launch are incomplete");
}

DDPConfig::DDPConfig(const std::vector<int> &device_ids, const std::string &backend, int rank, int world_size)
    : device_ids(device_ids), backend(backend), rank(rank), world_size(world_size) {}

DDPSequential::DDPSequential(std::shared_ptr<Sequential> model, const DDPConfig &config, bool average)
    : model(model), config(config), average(average) {
    if (config.backend != "nccl") LOG(LogLevel::ERROR, "Unsupported backend: " + config.backend);
    if (config.device_ids.empty()) LOG(LogLevel::ERROR, "DDP requires at least 1 device id.");
    const int world = static_cast<int>(config.device_ids.size());
    int rank = config.rank;
    // launched without MPI: a script that leaves DDPConfig's rank at its default gets it from the launcher's environment
    if (const char *r = std::getenv("RANK")) {
        const char *w = std::getenv("WORLD_SIZE");
        if (w && std::atoi(w) == world && config.rank == 0 && config.world_size <= 1) rank = std::atoi(r);
    }
    if (rank < 0 || rank >= world) LOG(LogLevel::ERROR, "DDP rank out of range: " + std::to_string(rank));
    this->config.rank = rank;
    this->config.world_size = world;
    const int device = config.device_ids[rank];
    cudaSetDevice(device);
    communicator = std::make_unique<B200Communicator>(rank, world, device, rendezvous_path());

    model->to_device("cuda:" + std::to_string(device));
    // Conv2d layers create their parameters lazily; make them exist before they are broadcast and registered
    model->preinit_layer();
    this->sync_base_parameters();

    // register every parameter-delta tensor once, in backward order, and cut the list into buckets
    g_registered.clear();
    g_average = average;
    for (BaseLayerCuda *l : parameter_layers_backward(*model)) {
        std::vector<std::pair<float *, size_t>> t = {{l->d_delta_mu_w, l->num_weights}, {l->d_delta_var_w, l->num_weights}};
        if (l->bias && l->num_biases > 0) {
            t.push_back({l->d_delta_mu_b, l->num_biases});
            t.push_back({l->d_delta_var_b, l->num_biases});
        }
        for (auto &x : t) {
            if (!x.first) LOG(LogLevel::ERROR, "DDP: a layer has no parameter-delta buffer (model not in training mode?)");
            const int idx = comm().tagi_comm_register(x.first, x.second);
            if (idx < 0) LOG(LogLevel::ERROR, std::string("tagi_comm_register: ") + comm().tagi_comm_last_error_string());
            g_registered[x.first] = idx;
        }
    }
    const char *mb = std::getenv("TAGI_B200_BUCKET_MB");
    require_ok(comm().tagi_comm_finalize_buckets((size_t)(mb ? std::atoi(mb) : 32) << 20), "tagi_comm_finalize_buckets");
}

void DDPSequential::sync_parameters() {
    // buckets whose tensors were all announced from backward() are already in flight; launch the rest, then make the
    // default stream (where the update runs) wait for all of them
    require_ok(comm().tagi_comm_flush(nullptr, this->average ? 1 : 0), "tagi_comm_flush");
    require_ok(comm().tagi_comm_wait(nullptr), "tagi_comm_wait");
}

void DDPSequential::sync_base_parameters() {
    for (BaseLayerCuda *l : parameter_layers_backward(*model)) {
        communicator->broadcast(l->d_mu_w, l->num_weights, 0);
        communicator->broadcast(l->d_var_w, l->num_weights, 0);
        if (l->bias && l->num_biases > 0) {
            communicator->broadcast(l->d_mu_b, l->num_biases, 0);
            communicator->broadcast(l->d_var_b, l->num_biases, 0);
        }
    }
}

void DDPSequential::forward(const std::vector<float> &mu_a, const std::vector<float> &var_a) {
    model->forward(mu_a, var_a);
}

void DDPSequential::backward() { model->backward(); }

void DDPSequential::step() {
    this->sync_parameters();
    model->step();
    communicator->check_async_error();
    tagi_b200_raise_on_kernel_abort();
}

void DDPSequential::train() { model->train(); }

void DDPSequential::eval() { model->eval(); }

void DDPSequential::barrier() { communicator->barrier(); }
