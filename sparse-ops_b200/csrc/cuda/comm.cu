// comm.cu -- communicator for the row-sharded paths: one process per GPU, NCCL over NVLink.
//
// The reference has no multi-device code; its row loop (src/ellpack_matmul.cpp:26) is what gets
// split.  Rank g owns rows [g*m/G, (g+1)*m/G) of E and computes its slab of Y locally; because Y
// is row-major, the slab of rank g is the contiguous range Y + g*rows*ld, so the exchange step is
// one in-place ncclAllGather and the gathered buffer is directly the next layer's X.
//
// NCCL is bound at run time with dlopen("libnccl.so.2"): inside a PyTorch process this resolves
// to the copy torch has already loaded, so both use one NCCL; there is no link-time dependency.
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

struct spx_comm {
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1, device = 0;
    float* token = nullptr;      // one float, operand of the barrier's all-reduce
};

namespace {

struct NcclApi {
    void* lib = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

NcclApi& api()
{
    static NcclApi a;
    static std::once_flag once;
    std::call_once(once, [] {
        a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!a.lib) a.lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!a.lib) return;
        a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(dlsym(a.lib, "ncclGetUniqueId"));
        a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(dlsym(a.lib, "ncclCommInitRank"));
        a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(dlsym(a.lib, "ncclCommDestroy"));
        a.AllGather = reinterpret_cast<decltype(a.AllGather)>(dlsym(a.lib, "ncclAllGather"));
        a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(dlsym(a.lib, "ncclAllReduce"));
        a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(dlsym(a.lib, "ncclGetErrorString"));
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllGather && a.AllReduce && a.GetErrorString;
    });
    return a;
}

int need_api()
{
    if (!api().ok) return spx::fail(SPX_ERR_COMM, "libnccl.so.2 could not be loaded: %s", dlerror() ? dlerror() : "missing symbols");
    return SPX_OK;
}

}  // namespace

static_assert(sizeof(ncclUniqueId) == SPX_UNIQUE_ID_BYTES, "ncclUniqueId size");

extern "C" {

int spx_comm_unique_id(char id[SPX_UNIQUE_ID_BYTES])
{
    if (!id) return spx::fail(SPX_ERR_ARG, "id is null");
    int rc = need_api();
    if (rc != SPX_OK) return rc;
    ncclUniqueId u;
    ncclResult_t r = api().GetUniqueId(&u);
    if (r != ncclSuccess) return spx::fail(SPX_ERR_COMM, "ncclGetUniqueId: %s", api().GetErrorString(r));
    memcpy(id, &u, SPX_UNIQUE_ID_BYTES);
    return SPX_OK;
}

int spx_comm_create(int rank, int world, const char id[SPX_UNIQUE_ID_BYTES], spx_comm** out)
{
    if (!out || !id) return spx::fail(SPX_ERR_ARG, "out / id is null");
    *out = nullptr;
    if (world < 1 || rank < 0 || rank >= world) return spx::fail(SPX_ERR_ARG, "bad rank %d of %d", rank, world);
    int rc = need_api();
    if (rc != SPX_OK) return rc;
    int device = 0;
    SPX_CUDA(cudaGetDevice(&device));
    spx_comm* c = new spx_comm();
    c->rank = rank;
    c->world = world;
    c->device = device;
    ncclUniqueId u;
    memcpy(&u, id, SPX_UNIQUE_ID_BYTES);
    ncclResult_t r = api().CommInitRank(&c->comm, world, u, rank);
    if (r != ncclSuccess) {
        delete c;
        return spx::fail(SPX_ERR_COMM, "ncclCommInitRank: %s", api().GetErrorString(r));
    }
    cudaError_t err = cudaMalloc(&c->token, sizeof(float));
    if (err == cudaSuccess) err = cudaMemset(c->token, 0, sizeof(float));
    if (err != cudaSuccess) {
        api().CommDestroy(c->comm);
        delete c;
        return spx::fail(SPX_ERR_CUDA, "communicator: token allocation failed: %s", cudaGetErrorString(err));
    }
    *out = c;
    return SPX_OK;
}

int spx_comm_info(const spx_comm* c, int* rank, int* world)
{
    if (!c) return spx::fail(SPX_ERR_ARG, "communicator is null");
    if (rank) *rank = c->rank;
    if (world) *world = c->world;
    return SPX_OK;
}

int spx_comm_barrier(spx_comm* c, void* stream)
{
    if (!c || !c->comm) return spx::fail(SPX_ERR_ARG, "communicator is null");
    ncclResult_t r = api().AllReduce(c->token, c->token, 1, ncclFloat, ncclSum, c->comm, (cudaStream_t)stream);
    if (r != ncclSuccess) return spx::fail(SPX_ERR_COMM, "ncclAllReduce: %s", api().GetErrorString(r));
    return SPX_OK;
}

int spx_comm_destroy(spx_comm* c)
{
    if (!c) return SPX_OK;
    cudaFree(c->token);
    if (c->comm && api().ok) api().CommDestroy(c->comm);
    delete c;
    return SPX_OK;
}

int spx_allgather_rows(spx_comm* c, float* Y, uint64_t rows_per_rank, uint64_t ld, void* stream)
{
    if (!c || !c->comm) return spx::fail(SPX_ERR_ARG, "communicator is null");
    const uint64_t count = rows_per_rank * ld;
    if (count == 0) return SPX_OK;
    if (!Y) return spx::fail(SPX_ERR_ARG, "Y is null");
    ncclResult_t r = api().AllGather(Y + (size_t)c->rank * count, Y, count, ncclFloat, c->comm, (cudaStream_t)stream);
    if (r != ncclSuccess) return spx::fail(SPX_ERR_COMM, "ncclAllGather: %s", api().GetErrorString(r));
    return SPX_OK;
}

}  // extern "C"
