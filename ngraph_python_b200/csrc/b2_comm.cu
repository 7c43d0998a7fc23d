// Gradient allreduce over NCCL (NVLink 5 / NVSwitch) behind the C ABI.
//
// Takes the place of hetr's GPU allreduce, CudaAllReduceKernel (ngraph/transformers/gpu/
// tensor_ops.py:428-618): per tensor a reduce-scatter by peer-to-peer memcpy, a float_accum
// kernel, an all-gather by peer-to-peer memcpy, three MPI barriers and host synchronisations.
// Here one process per GPU holds one NCCL communicator; a bucket of gradients is reduced in place
// by ONE ncclAllReduce on the stream the caller names (its communication stream), so the exchange
// runs beside back-propagation; 'mean' divides by the number of replicas in a small kernel on the
// same stream (the reference's kernel divides too, tensor_ops.py:95-108).  Errors NCCL reports
// asynchronously (a peer that died, a link fault) are polled, not waited for: b2_comm_poll_error
// turns them into B2_ERR_COMM so the host can stop instead of hanging in a synchronisation, and
// b2_comm_abort ends what is in flight.
//
// NCCL is loaded at run time (the copy already in the process -- PyTorch brings one -- else
// libnccl.so.2 from the loader path or from b2_set_nccl_path); the library has no link-time
// dependency on it and everything else works without it.
#include <dlfcn.h>

#include <cstring>
#include <mutex>
#include <string>

#include "b2_common.h"

namespace {

typedef struct ncclComm* ncclComm_t;
struct NcclId { char internal[B2_COMM_ID_BYTES]; };
const int kNcclFloat32 = 7, kNcclSum = 0, kNcclSuccess = 0, kNcclInProgress = 7;

struct Nccl {
    void* handle = nullptr;
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, NcclId, int) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
    int (*CommAbort)(ncclComm_t) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    int (*GetVersion)(int*) = nullptr;
};

Nccl g_nccl;
std::string g_nccl_dir;
std::mutex g_nccl_mutex;

int load_nccl() {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.handle) return B2_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);      // the copy already loaded
    if (!h && !g_nccl_dir.empty()) h = dlopen((g_nccl_dir + "/libnccl.so.2").c_str(), RTLD_NOW);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW);
    if (!h) return b2::fail(B2_ERR_UNAVAILABLE, "libnccl.so.2 could not be loaded: %s", dlerror());
#define B2_SYM(field, name)                                                                  \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name));                \
    if (!g_nccl.field) return b2::fail(B2_ERR_UNAVAILABLE, "libnccl.so.2 lacks %s", name)
    B2_SYM(GetUniqueId, "ncclGetUniqueId");
    B2_SYM(CommInitRank, "ncclCommInitRank");
    B2_SYM(AllReduce, "ncclAllReduce");
    B2_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
    B2_SYM(CommAbort, "ncclCommAbort");
    B2_SYM(CommDestroy, "ncclCommDestroy");
    B2_SYM(GetErrorString, "ncclGetErrorString");
    B2_SYM(GetVersion, "ncclGetVersion");
#undef B2_SYM
    g_nccl.handle = h;
    return B2_OK;
}

int comm_fail(const char* what, int rc) {
    return b2::fail(B2_ERR_COMM, "%s: %s", what,
                    g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "NCCL error");
}

__global__ void __launch_bounds__(256) scale_kernel(float* buf, long long n, float f) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        buf[i] *= f;
}

}  // namespace

struct b2_comm {
    ncclComm_t comm;
    int rank, nranks, device;
    bool dead;
};

extern "C" int b2_set_nccl_path(const char* path) {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    g_nccl_dir = path ? path : "";
    return B2_OK;
}

extern "C" int b2_comm_version(int32_t* version) {
    B2_REQUIRE(version, "null argument");
    int rc = load_nccl();
    if (rc) return rc;
    int v = 0;
    if ((rc = g_nccl.GetVersion(&v)) != kNcclSuccess) return comm_fail("ncclGetVersion", rc);
    *version = v;
    return B2_OK;
}

extern "C" int b2_comm_unique_id(void* id_out) {
    B2_REQUIRE(id_out, "null argument");
    int rc = load_nccl();
    if (rc) return rc;
    NcclId id;
    if ((rc = g_nccl.GetUniqueId(&id)) != kNcclSuccess) return comm_fail("ncclGetUniqueId", rc);
    memcpy(id_out, &id, sizeof(id));
    return B2_OK;
}

extern "C" int b2_comm_init(const void* id, int32_t rank, int32_t nranks, int32_t device,
                            b2_comm** out) {
    B2_REQUIRE(id && out && nranks >= 1 && rank >= 0 && rank < nranks, "bad argument");
    int rc = load_nccl();
    if (rc) return rc;
    B2_CUDA(cudaSetDevice(device));
    NcclId nid;
    memcpy(&nid, id, sizeof(nid));
    ncclComm_t c = nullptr;
    if ((rc = g_nccl.CommInitRank(&c, nranks, nid, rank)) != kNcclSuccess)
        return comm_fail("ncclCommInitRank", rc);
    b2_comm* h = new b2_comm;
    h->comm = c; h->rank = rank; h->nranks = nranks; h->device = device; h->dead = false;
    *out = h;
    return B2_OK;
}

extern "C" int b2_comm_allreduce_f32(b2_comm* c, float* buf, int64_t count, int32_t mean,
                                     void* stream) {
    B2_REQUIRE(c && buf && count >= 0, "bad argument");
    if (c->dead) return b2::fail(B2_ERR_COMM, "the communicator has been aborted");
    if (count == 0) return B2_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int rc = g_nccl.AllReduce(buf, buf, (size_t)count, kNcclFloat32, kNcclSum, c->comm, st);
    if (rc != kNcclSuccess) return comm_fail("ncclAllReduce", rc);
    if (mean && c->nranks > 1) {
        long long blocks = (count + 255) / 256;
        if (blocks > 148 * 8) blocks = 148 * 8;
        scale_kernel<<<(unsigned)blocks, 256, 0, st>>>(buf, count, 1.0f / (float)c->nranks);
        B2_CUDA(cudaGetLastError());
    }
    return B2_OK;
}

extern "C" int b2_comm_poll_error(b2_comm* c) {
    B2_REQUIRE(c, "bad argument");
    if (c->dead) return b2::fail(B2_ERR_COMM, "the communicator has been aborted");
    int async = kNcclSuccess;
    const int rc = g_nccl.CommGetAsyncError(c->comm, &async);
    if (rc != kNcclSuccess) return comm_fail("ncclCommGetAsyncError", rc);
    if (async != kNcclSuccess && async != kNcclInProgress)
        return comm_fail("a collective failed asynchronously", async);
    return B2_OK;
}

extern "C" int b2_comm_abort(b2_comm* c) {
    B2_REQUIRE(c, "bad argument");
    if (!c->dead) {
        c->dead = true;
        const int rc = g_nccl.CommAbort(c->comm);
        if (rc != kNcclSuccess) return comm_fail("ncclCommAbort", rc);
    }
    return B2_OK;
}

extern "C" int b2_comm_destroy(b2_comm* c) {
    if (!c) return B2_OK;
    int rc = kNcclSuccess;
    if (!c->dead) rc = g_nccl.CommDestroy(c->comm);
    delete c;
    if (rc != kNcclSuccess) return comm_fail("ncclCommDestroy", rc);
    return B2_OK;
}
