// Data-parallel exchange of TAGI parameter deltas over NCCL (see include/tagi_b200_comm.h).
// Host-only C++: the collectives are NCCL's; what this file adds is the MPI-free rendezvous, the bucket plan and the
// event-ordered overlap with the backward pass.
#include <cuda_runtime.h>
#include <fcntl.h>
#include <nccl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <algorithm>
#include <vector>

#include "../../include/tagi_b200.h"
#include "../../include/tagi_b200_comm.h"

namespace {

thread_local std::string g_err;
int fail(int code, const std::string &m) {
    g_err = m;
    return code;
}
#define CU(expr)                                                                                   \
    do {                                                                                           \
        cudaError_t e__ = (expr);                                                                  \
        if (e__ != cudaSuccess) return fail(TAGI_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e__)); \
    } while (0)
#define NC(expr)                                                                                   \
    do {                                                                                           \
        ncclResult_t r__ = (expr);                                                                 \
        if (r__ != ncclSuccess && r__ != ncclInProgress)                                           \
            return fail(TAGI_ERR_COMM, std::string(#expr) + ": " + ncclGetErrorString(r__));       \
    } while (0)

struct Tensor {
    float *ptr;
    size_t count;
    int bucket;
};
struct Run {   // tensors of a bucket that lie back to back in memory: exchanged as one allreduce
    float *ptr;
    size_t count;
};
struct Bucket {
    std::vector<int> tensors;
    std::vector<Run> runs;   // filled when every rank found the same runs (see tagi_comm_finalize_buckets)
    int ready = 0;       // tensors marked ready in this step
    bool launched = false;
    cudaEvent_t done = nullptr;
};
struct Comm {
    ncclComm_t nccl = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev = nullptr;  // compute -> comm ordering
    float *token = nullptr;    // one float for tagi_comm_barrier
    int rank = 0, world = 1, device = 0;
    bool finalized = false;
    std::vector<Tensor> tensors;
    std::vector<Bucket> buckets;
    std::vector<char> ready;   // per tensor, this step
};
Comm *g = nullptr;
int g_max_ctas = 0;  // 0: NCCL's default; else the upper bound on the CTAs one NCCL kernel may use (tagi_comm_set_max_ctas)

// What travels through the rendezvous file of tagi_comm_init_file: enough to tell this job's id from a file that an
// earlier job left at the same path.
struct RendezvousBlob {
    char magic[8];
    int world;
    int pid;
    long long unix_ms;  // when rank 0 wrote it
    unsigned char id[TAGI_COMM_ID_BYTES];
};
long long now_unix_ms() {
    return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::system_clock::now().time_since_epoch()).count();
}

int need_comm() { return g ? TAGI_OK : fail(TAGI_ERR_COMM, "communicator not initialised"); }

int launch_bucket(Bucket &b, cudaStream_t compute, int average) {
    if (b.launched) return TAGI_OK;
    CU(cudaEventRecord(g->ev, compute));
    CU(cudaStreamWaitEvent(g->stream, g->ev, 0));
    NC(ncclGroupStart());
    if (!b.runs.empty()) {
        for (const Run &r : b.runs)
            NC(ncclAllReduce(r.ptr, r.ptr, r.count, ncclFloat32, average ? ncclAvg : ncclSum, g->nccl, g->stream));
    } else {
        for (int t : b.tensors) {
            Tensor &x = g->tensors[t];
            NC(ncclAllReduce(x.ptr, x.ptr, x.count, ncclFloat32, average ? ncclAvg : ncclSum, g->nccl, g->stream));
        }
    }
    NC(ncclGroupEnd());
    CU(cudaEventRecord(b.done, g->stream));
    b.launched = true;
    return TAGI_OK;
}

}  // namespace

extern "C" {

const char *tagi_comm_last_error_string(void) { return g_err.c_str(); }

// ------------------------------------------------------------------------------------------------ host-only pieces
int tagi_rendezvous_publish(const char *path, const void *blob, size_t bytes) {
    if (!path || !blob || bytes == 0) return fail(TAGI_ERR_INVALID_ARGUMENT, "rendezvous: null path or empty blob");
    const std::string tmp = std::string(path) + ".tmp." + std::to_string((long)getpid());
    FILE *f = std::fopen(tmp.c_str(), "wb");
    if (!f) return fail(TAGI_ERR_COMM, "rendezvous: cannot create " + tmp);
    const size_t w = std::fwrite(blob, 1, bytes, f);
    std::fclose(f);
    if (w != bytes) return fail(TAGI_ERR_COMM, "rendezvous: short write to " + tmp);
    if (std::rename(tmp.c_str(), path) != 0) return fail(TAGI_ERR_COMM, std::string("rendezvous: cannot rename to ") + path);
    return TAGI_OK;
}

int tagi_rendezvous_fetch(const char *path, void *blob, size_t bytes, int timeout_ms) {
    if (!path || !blob || bytes == 0) return fail(TAGI_ERR_INVALID_ARGUMENT, "rendezvous: null path or empty blob");
    const auto t0 = std::chrono::steady_clock::now();
    while (true) {
        FILE *f = std::fopen(path, "rb");
        if (f) {
            const size_t r = std::fread(blob, 1, bytes, f);
            std::fclose(f);
            if (r == bytes) return TAGI_OK;
        }
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms > timeout_ms)
            return fail(TAGI_ERR_COMM, std::string("rendezvous: nothing published at ") + path + " within " +
                                           std::to_string(timeout_ms) + " ms (did rank 0 start?)");
        std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
}

int tagi_comm_plan_buckets(const size_t *counts, int n, size_t bucket_bytes, int *bucket_of) {
    if (!counts || !bucket_of || n < 0 || bucket_bytes == 0) {
        fail(TAGI_ERR_INVALID_ARGUMENT, "plan_buckets: bad arguments");
        return -TAGI_ERR_INVALID_ARGUMENT;
    }
    int bucket = 0;
    size_t used = 0;
    for (int i = 0; i < n; i++) {
        const size_t bytes = counts[i] * sizeof(float);
        if (used > 0 && used + bytes > bucket_bytes) {
            bucket++;
            used = 0;
        }
        bucket_of[i] = bucket;
        used += bytes;
    }
    return n == 0 ? 0 : bucket + 1;
}

// ------------------------------------------------------------------------------------------------ communicator
int tagi_comm_create_id(void *id) {
    if (!id) return fail(TAGI_ERR_INVALID_ARGUMENT, "null id");
    static_assert(sizeof(ncclUniqueId) == TAGI_COMM_ID_BYTES, "ncclUniqueId size");
    ncclUniqueId u;
    NC(ncclGetUniqueId(&u));
    std::memcpy(id, &u, sizeof(u));
    return TAGI_OK;
}

int tagi_comm_init(const void *id, int rank, int world_size, int device) {
    if (g) return fail(TAGI_ERR_COMM, "communicator already initialised");
    if (!id || world_size < 1 || rank < 0 || rank >= world_size)
        return fail(TAGI_ERR_INVALID_ARGUMENT, "comm_init: bad id, rank or world size");
    CU(cudaSetDevice(device));
    Comm *c = new Comm;
    c->rank = rank, c->world = world_size, c->device = device;
    ncclUniqueId u;
    std::memcpy(&u, id, sizeof(u));
    ncclResult_t r;
    if (g_max_ctas > 0) {
        // bound the SMs NCCL's kernels take from the compute kernels they overlap
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.maxCTAs = g_max_ctas;
        r = ncclCommInitRankConfig(&c->nccl, world_size, u, rank, &cfg);
    } else {
        r = ncclCommInitRank(&c->nccl, world_size, u, rank);
    }
    if (r != ncclSuccess) {
        delete c;
        return fail(TAGI_ERR_COMM, std::string("ncclCommInitRank: ") + ncclGetErrorString(r));
    }
    cudaError_t e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->ev, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        ncclCommAbort(c->nccl);
        delete c;
        return fail(TAGI_ERR_CUDA, std::string("comm stream/event: ") + cudaGetErrorString(e));
    }
    g = c;
    return TAGI_OK;
}

int tagi_rendezvous_publish_id(const char *path, const void *id, int world_size) {
    if (!path || !id) return fail(TAGI_ERR_INVALID_ARGUMENT, "rendezvous: null path or id");
    RendezvousBlob blob;
    std::memset(&blob, 0, sizeof(blob));
    std::memcpy(blob.magic, "TAGIRDV1", 8);
    blob.world = world_size, blob.pid = (int)getpid(), blob.unix_ms = now_unix_ms();
    std::memcpy(blob.id, id, TAGI_COMM_ID_BYTES);
    ::unlink(path);  // whatever an earlier job left there
    return tagi_rendezvous_publish(path, &blob, sizeof(blob));
}

int tagi_rendezvous_fetch_id(const char *path, void *id, int world_size, int timeout_ms) {
    if (!path || !id) return fail(TAGI_ERR_INVALID_ARGUMENT, "rendezvous: null path or id");
    // A file that an earlier job left at this path is told apart by its header: wrong magic or world size, or written
    // more than timeout_ms before this rank started waiting. Such a file is skipped and the wait goes on until rank 0
    // replaces it or the deadline passes.
    RendezvousBlob blob;
    const long long started = now_unix_ms();
    while (true) {
        const long long left = (long long)timeout_ms - (now_unix_ms() - started);
        if (left <= 0)
            return fail(TAGI_ERR_COMM, std::string("rendezvous: no id of this job at ") + path + " within " +
                                           std::to_string(timeout_ms) + " ms (did rank 0 start?)");
        int rc = tagi_rendezvous_fetch(path, &blob, sizeof(blob), (int)left);
        if (rc != TAGI_OK) return rc;
        if (!std::memcmp(blob.magic, "TAGIRDV1", 8) && blob.world == world_size &&
            blob.unix_ms >= started - (long long)timeout_ms)
            break;
        std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
    std::memcpy(id, blob.id, TAGI_COMM_ID_BYTES);
    return TAGI_OK;
}

int tagi_comm_init_file(const char *path, int rank, int world_size, int device, int timeout_ms) {
    unsigned char id[TAGI_COMM_ID_BYTES];
    int rc;
    if (rank == 0) {
        if ((rc = tagi_comm_create_id(id)) != TAGI_OK) return rc;
        if ((rc = tagi_rendezvous_publish_id(path, id, world_size)) != TAGI_OK) return rc;
    } else {
        if ((rc = tagi_rendezvous_fetch_id(path, id, world_size, timeout_ms)) != TAGI_OK) return rc;
    }
    rc = tagi_comm_init(id, rank, world_size, device);
    // ncclCommInitRank returns once every rank has joined: nobody needs the file any more
    if (rc == TAGI_OK && rank == 0) ::unlink(path);
    return rc;
}

int tagi_comm_set_max_ctas(int max_ctas) {
    if (max_ctas < 0 || max_ctas > 64) return fail(TAGI_ERR_INVALID_ARGUMENT, "max_ctas must be 0 (NCCL default) .. 64");
    if (g) return fail(TAGI_ERR_COMM, "set_max_ctas must be called before the communicator is created");
    g_max_ctas = max_ctas;
    return TAGI_OK;
}

int tagi_comm_rank(void) { return g ? g->rank : 0; }
int tagi_comm_world_size(void) { return g ? g->world : 1; }

int tagi_comm_register(float *ptr, size_t count) {
    if (need_comm() != TAGI_OK) return -TAGI_ERR_COMM;
    if (g->finalized) {
        fail(TAGI_ERR_COMM, "register after finalize_buckets");
        return -TAGI_ERR_COMM;
    }
    if (!ptr || count == 0) {
        fail(TAGI_ERR_INVALID_ARGUMENT, "register: null pointer or zero count");
        return -TAGI_ERR_INVALID_ARGUMENT;
    }
    g->tensors.push_back({ptr, count, -1});
    return (int)g->tensors.size() - 1;
}

int tagi_comm_finalize_buckets(size_t bucket_bytes) {
    int rc = need_comm();
    if (rc != TAGI_OK) return rc;
    if (g->finalized) return fail(TAGI_ERR_COMM, "buckets already finalized");
    const int n = (int)g->tensors.size();
    std::vector<size_t> counts(n);
    std::vector<int> of(n);
    for (int i = 0; i < n; i++) counts[i] = g->tensors[i].count;
    const int nb = tagi_comm_plan_buckets(counts.data(), n, bucket_bytes, of.data());
    if (nb < 0) return -nb;
    g->buckets.resize(nb);
    for (int i = 0; i < n; i++) {
        g->tensors[i].bucket = of[i];
        g->buckets[of[i]].tensors.push_back(i);
    }
    for (auto &b : g->buckets) CU(cudaEventCreateWithFlags(&b.done, cudaEventDisableTiming));
    g->ready.assign(n, 0);
    g->finalized = true;
    // Tensors of a bucket that lie back to back in memory (a caller that carves its delta tensors out of one buffer)
    // travel as one allreduce: a network's many small tensors otherwise cost a collective each, and NCCL's bandwidth
    // falls with the message size (ResNet-18, 124 tensors in 3 buckets, 8 GPUs: 1.16 ms for 94 MB). Every rank must issue
    // the same sequence of collectives, so the runs are used only if all ranks found the same ones: a hash over the run
    // boundaries and the registration indices inside them is compared across the ranks (min == max).
    std::vector<std::vector<Run>> runs(nb);
    unsigned long long h = 1469598103934665603ull;
    auto mix = [&h](unsigned long long v) { h = (h ^ v) * 1099511628211ull; };
    bool any_merge = false;
    for (int bi = 0; bi < nb; bi++) {
        std::vector<int> order = g->buckets[bi].tensors;
        std::sort(order.begin(), order.end(), [](int a, int b) { return g->tensors[a].ptr < g->tensors[b].ptr; });
        mix(0xB0000000ull + (unsigned long long)bi);
        for (int t : order) {
            const Tensor &x = g->tensors[t];
            if (!runs[bi].empty() && runs[bi].back().ptr + runs[bi].back().count == x.ptr) {
                runs[bi].back().count += x.count;
                any_merge = true;
            } else {
                runs[bi].push_back(Run{x.ptr, x.count});
                mix(0xA0000000ull);   // a run starts here
            }
            mix((unsigned long long)t);
            mix((unsigned long long)x.count);
        }
    }
    unsigned long long *dev = nullptr;
    CU(cudaMalloc(&dev, 2 * sizeof(unsigned long long)));
    const unsigned long long mine[2] = {any_merge ? h : 0ull, any_merge ? h : ~0ull};   // a rank without merges vetoes
    CU(cudaMemcpyAsync(dev, mine, sizeof(mine), cudaMemcpyHostToDevice, g->stream));
    NC(ncclGroupStart());
    NC(ncclAllReduce(dev, dev, 1, ncclUint64, ncclMin, g->nccl, g->stream));
    NC(ncclAllReduce(dev + 1, dev + 1, 1, ncclUint64, ncclMax, g->nccl, g->stream));
    NC(ncclGroupEnd());
    unsigned long long agreed[2] = {0, 1};
    CU(cudaMemcpyAsync(agreed, dev, sizeof(agreed), cudaMemcpyDeviceToHost, g->stream));
    CU(cudaStreamSynchronize(g->stream));
    CU(cudaFree(dev));
    if (any_merge && agreed[0] == h && agreed[1] == h)
        for (int bi = 0; bi < nb; bi++) g->buckets[bi].runs = std::move(runs[bi]);
    return TAGI_OK;
}

int tagi_comm_num_collectives(void) {
    if (!g) return 0;
    int n = 0;
    for (const auto &b : g->buckets) n += (int)(b.runs.empty() ? b.tensors.size() : b.runs.size());
    return n;
}

int tagi_comm_num_buckets(void) { return g ? (int)g->buckets.size() : 0; }
int tagi_comm_num_tensors(void) { return g ? (int)g->tensors.size() : 0; }
int tagi_comm_bucket_of(int i) { return (g && i >= 0 && i < (int)g->tensors.size()) ? g->tensors[i].bucket : -1; }

int tagi_comm_tensor_ready(int i, void *compute_stream, int average) {
    int rc = need_comm();
    if (rc != TAGI_OK) return rc;
    if (!g->finalized) return fail(TAGI_ERR_COMM, "tensor_ready before finalize_buckets");
    if (i < 0 || i >= (int)g->tensors.size()) return fail(TAGI_ERR_INVALID_ARGUMENT, "tensor index out of range");
    if (g->ready[i]) return TAGI_OK;
    g->ready[i] = 1;
    Bucket &b = g->buckets[g->tensors[i].bucket];
    if (++b.ready == (int)b.tensors.size()) return launch_bucket(b, static_cast<cudaStream_t>(compute_stream), average);
    return TAGI_OK;
}

int tagi_comm_flush(void *compute_stream, int average) {
    int rc = need_comm();
    if (rc != TAGI_OK) return rc;
    if (!g->finalized) return fail(TAGI_ERR_COMM, "flush before finalize_buckets");
    for (auto &b : g->buckets)
        if ((rc = launch_bucket(b, static_cast<cudaStream_t>(compute_stream), average)) != TAGI_OK) return rc;
    return TAGI_OK;
}

int tagi_comm_wait(void *compute_stream) {
    int rc = need_comm();
    if (rc != TAGI_OK) return rc;
    for (auto &b : g->buckets) {
        if (b.launched) CU(cudaStreamWaitEvent(static_cast<cudaStream_t>(compute_stream), b.done, 0));
        b.launched = false;
        b.ready = 0;
    }
    std::fill(g->ready.begin(), g->ready.end(), 0);
    return TAGI_OK;
}

int tagi_comm_allreduce(float *ptr, size_t count, int average, void *compute_stream) {
    int rc = need_comm();
    if (rc != TAGI_OK) return rc;
    if (!ptr || count == 0) return fail(TAGI_ERR_INVALID_ARGUMENT, "allreduce: null pointer or zero count");
    cudaStream_t cs = static_cast<cudaStream_t>(compute_stream);
    CU(cudaEventRecord(g->ev, cs));
    CU(cudaStreamWaitEvent(g->stream, g->ev, 0));
    NC(ncclAllReduce(ptr, ptr, count, ncclFloat32, average ? ncclAvg : ncclSum, g->nccl, g->stream));
    CU(cudaEventRecord(g->ev, g->stream));
    CU(cudaStreamWaitEvent(cs, g->ev, 0));
    return TAGI_OK;
}

int tagi_comm_broadcast(float *ptr, size_t count, int root, void *compute_stream) {
    int rc = need_comm();
    if (rc != TAGI_OK) return rc;
    if (!ptr || count == 0 || root < 0 || root >= g->world)
        return fail(TAGI_ERR_INVALID_ARGUMENT, "broadcast: bad pointer, count or root");
    cudaStream_t cs = static_cast<cudaStream_t>(compute_stream);
    CU(cudaEventRecord(g->ev, cs));
    CU(cudaStreamWaitEvent(g->stream, g->ev, 0));
    NC(ncclBroadcast(ptr, ptr, count, ncclFloat32, root, g->nccl, g->stream));
    CU(cudaEventRecord(g->ev, g->stream));
    CU(cudaStreamWaitEvent(cs, g->ev, 0));
    return TAGI_OK;
}

int tagi_comm_check(void) {
    int rc = need_comm();
    if (rc != TAGI_OK) return rc;
    ncclResult_t async = ncclSuccess;
    ncclResult_t r = ncclCommGetAsyncError(g->nccl, &async);
    if (r != ncclSuccess) return fail(TAGI_ERR_COMM, std::string("ncclCommGetAsyncError: ") + ncclGetErrorString(r));
    if (async != ncclSuccess && async != ncclInProgress)
        return fail(TAGI_ERR_COMM, std::string("NCCL asynchronous error: ") + ncclGetErrorString(async));
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) return fail(TAGI_ERR_CUDA, std::string("CUDA error pending: ") + cudaGetErrorString(e));
    return TAGI_OK;
}

int tagi_comm_sync_stream(void) {
    int rc = need_comm();
    if (rc != TAGI_OK) return rc;
    CU(cudaStreamSynchronize(g->stream));
    return TAGI_OK;
}

int tagi_comm_barrier(void) {
    int rc = need_comm();
    if (rc != TAGI_OK) return rc;
    // an allreduce of one float that every rank must enter, then a host wait for it: no rank returns before all arrived
    if (!g->token) CU(cudaMalloc(&g->token, sizeof(float)));
    CU(cudaMemsetAsync(g->token, 0, sizeof(float), g->stream));
    NC(ncclAllReduce(g->token, g->token, 1, ncclFloat32, ncclSum, g->nccl, g->stream));
    CU(cudaStreamSynchronize(g->stream));
    return TAGI_OK;
}

int tagi_comm_destroy(void) {
    if (!g) return TAGI_OK;
    cudaStreamSynchronize(g->stream);
    for (auto &b : g->buckets)
        if (b.done) cudaEventDestroy(b.done);
    if (g->ev) cudaEventDestroy(g->ev);
    if (g->token) cudaFree(g->token);
    if (g->stream) cudaStreamDestroy(g->stream);
    if (g->nccl) ncclCommDestroy(g->nccl);
    delete g;
    g = nullptr;
    return TAGI_OK;
}

}  // extern "C"
