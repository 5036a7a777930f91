// Data-parallel glue: sequences are independent, so ranks own disjoint blocks
// of sequences and the only exchange is one all-reduce (sum) of
// {loss_sum, n_valid} - 16 bytes - over NCCL.  mean = sum(loss) / sum(n_valid)
// then matches the reference's single-process mean (src/model.rs:3253-3257).
//
// NCCL is resolved at run time (dlopen of libnccl.so.2, which is already in
// the process when PyTorch is) so the library has no link-time dependency on
// a particular NCCL build.  The reference has no distributed layer.
#include <dlfcn.h>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <chrono>
#include <cstring>
#include <string>
#include <thread>

#include "common.hpp"

namespace ullis {

typedef struct ncclComm* ncclComm_t;
struct UniqueId { char internal[128]; };

struct NcclApi {
    void* handle = nullptr;
    int (*GetUniqueId)(UniqueId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

struct NcclState {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    double* dev = nullptr;  // 2 doubles
};

static NcclApi& api() {
    static NcclApi a;
    if (a.handle) return a;
    const char* names[] = {getenv("ULLIS_CUDA_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        if (!n || !*n) continue;
        a.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (a.handle) break;
    }
    if (!a.handle) fail(ULLIS_CUDA_ERR_NCCL, std::string("cannot load libnccl.so.2: ") + dlerror());
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(a.handle, "ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(a.handle, "ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(a.handle, "ncclCommDestroy"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(a.handle, "ncclAllReduce"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(a.handle, "ncclGetErrorString"));
    if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllReduce || !a.GetErrorString) {
        a.handle = nullptr;
        fail(ULLIS_CUDA_ERR_NCCL, "libnccl.so.2 lacks a required symbol");
    }
    return a;
}

static void nccl_check(int rc, const char* what) {
    if (rc != 0) fail(ULLIS_CUDA_ERR_NCCL, std::string(what) + ": " + api().GetErrorString(rc));
}

void dp_allreduce_device(ullis_cuda_runtime* rt, double* dev, size_t count) {
    if (!rt->nccl) fail(ULLIS_CUDA_ERR_NCCL, "data-parallel group is not initialised");
    nccl_check(api().AllReduce(dev, dev, count, /*ncclDouble*/ 8, /*ncclSum*/ 0, rt->nccl->comm, rt->stream),
               "ncclAllReduce");
}

}  // namespace ullis

using namespace ullis;

static std::string g_dp_error;

extern "C" {

int32_t ullis_cuda_dp_unique_id(uint8_t id[128]) {
    try {
        if (!id) fail(ULLIS_CUDA_ERR_ARG, "id is null");
        UniqueId u;
        nccl_check(api().GetUniqueId(&u), "ncclGetUniqueId");
        memcpy(id, u.internal, 128);
        return ULLIS_CUDA_OK;
    } catch (const Error& e) {
        g_dp_error = e.msg;
        set_global_error(e.msg.c_str());
        return e.code;
    }
}

int32_t ullis_cuda_dp_rendezvous(const char* dir, const char* tag, int32_t rank, int32_t world, uint32_t timeout_ms) {
    try {
        if (!dir || !tag || !*dir || !*tag || world < 1 || rank < 0 || rank >= world)
            fail(ULLIS_CUDA_ERR_ARG, "bad rendezvous directory / tag / rank / world");
        const std::string base = std::string(dir) + "/" + tag + ".";
        const int fd = open((base + std::to_string(rank)).c_str(), O_CREAT | O_WRONLY, 0644);
        if (fd < 0) fail(ULLIS_CUDA_ERR_ARG, "cannot create the rendezvous file of rank " + std::to_string(rank) +
                                                 " in " + dir + ": " + strerror(errno));
        close(fd);
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
        for (;;) {
            int missing = -1;
            for (int r = 0; r < world && missing < 0; ++r) {
                struct stat st;
                if (stat((base + std::to_string(r)).c_str(), &st) != 0) missing = r;
            }
            if (missing < 0) return ULLIS_CUDA_OK;
            if (std::chrono::steady_clock::now() >= deadline)
                fail(ULLIS_CUDA_ERR_TIMEOUT, "data-parallel rendezvous timed out after " + std::to_string(timeout_ms) +
                                                 " ms: rank " + std::to_string(missing) + " of " +
                                                 std::to_string(world) + " never arrived");
            std::this_thread::sleep_for(std::chrono::milliseconds(5));
        }
    } catch (const Error& e) {
        set_global_error(e.msg.c_str());
        return e.code;
    }
}

int32_t ullis_cuda_dp_init(ullis_cuda_runtime* rt, int32_t rank, int32_t world, const uint8_t id[128]) {
    if (!rt) return ULLIS_CUDA_ERR_ARG;
    try {
        if (!id || world < 1 || rank < 0 || rank >= world) fail(ULLIS_CUDA_ERR_ARG, "bad rank / world / id");
        if (rt->nccl) fail(ULLIS_CUDA_ERR_ARG, "data-parallel group already initialised");
        rt->bind();
        UniqueId u;
        memcpy(u.internal, id, 128);
        NcclState* st = new NcclState();
        st->rank = rank;
        st->world = world;
        int rc = api().CommInitRank(&st->comm, world, u, rank);
        if (rc != 0) {
            delete st;
            nccl_check(rc, "ncclCommInitRank");
        }
        cudaError_t ce = cudaMalloc(&st->dev, 16);
        if (ce != cudaSuccess) {
            api().CommDestroy(st->comm);
            delete st;
            fail(ULLIS_CUDA_ERR_NOMEM, "cudaMalloc failed");
        }
        rt->nccl = st;
        return ULLIS_CUDA_OK;
    } catch (const Error& e) {
        rt->last_error = e.msg;
        return e.code;
    }
}

int32_t ullis_cuda_dp_allreduce_loss(ullis_cuda_runtime* rt, double* loss_sum, uint64_t* n_valid) {
    if (!rt) return ULLIS_CUDA_ERR_ARG;
    try {
        if (!loss_sum || !n_valid) fail(ULLIS_CUDA_ERR_ARG, "loss_sum / n_valid is null");
        if (!rt->nccl) fail(ULLIS_CUDA_ERR_NCCL, "data-parallel group is not initialised");
        rt->bind();
        NcclState* st = rt->nccl;
        // n_valid travels as a double: exact up to 2^53 positions
        double host[2] = {*loss_sum, (double)*n_valid};
        rt->h2d(st->dev, host, 16);
        nccl_check(api().AllReduce(st->dev, st->dev, 2, /*ncclDouble*/ 8, /*ncclSum*/ 0, st->comm, rt->stream),
                   "ncclAllReduce");
        rt->d2h(host, st->dev, 16);
        rt->sync();
        *loss_sum = host[0];
        *n_valid = (uint64_t)(host[1] + 0.5);
        return ULLIS_CUDA_OK;
    } catch (const Error& e) {
        rt->last_error = e.msg;
        return e.code;
    }
}

int32_t ullis_cuda_dp_finalize(ullis_cuda_runtime* rt) {
    if (!rt) return ULLIS_CUDA_ERR_ARG;
    if (!rt->nccl) return ULLIS_CUDA_OK;
    NcclState* st = rt->nccl;
    rt->nccl = nullptr;
    cudaSetDevice(rt->device);
    if (st->dev) cudaFree(st->dev);
    int rc = 0;
    try {
        rc = api().CommDestroy(st->comm);
    } catch (const Error&) {
        rc = 1;
    }
    delete st;
    return rc == 0 ? ULLIS_CUDA_OK : ULLIS_CUDA_ERR_NCCL;
}

}  // extern "C"
