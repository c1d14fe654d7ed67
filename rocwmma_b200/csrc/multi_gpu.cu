// Multi-GPU plumbing of the C ABI: one process per GPU, NCCL for the only exchange the sharded paths need (the
// broadcast of the operand every rank uses whole: A of a column-sharded GEMM, x of a row-sharded GEMV), and the
// arithmetic of the shards themselves.  The reference has no multi-GPU path; the sharding rules are those of
// rocwmma_b200/sharding.py.
//
// NCCL is opened at run time (the library already in the process if there is one, e.g. the one PyTorch brought, else
// libnccl.so.2 from the loader path), so librocwmma_b200.so itself does not depend on it; without NCCL the
// b200wmma_mg_* calls return B200WMMA_ERR_UNSUPPORTED.  The environment variable B200WMMA_NCCL_LIBRARY, read once at
// the first b200wmma_mg_* call, names another library file to open instead (a full path or a name for the loader).
#include "common.cuh"

#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <mutex>
#include <new>
#include <string>

namespace
{
    // the part of NCCL's C API used here (nccl.h: ncclUniqueId is 128 opaque bytes, ncclResult_t 0 = success)
    struct NcclId
    {
        char internal[128];
    };
    static_assert(sizeof(NcclId) == B200WMMA_MG_ID_BYTES, "unique id size");
    using GetUniqueIdFn = int (*)(NcclId*);
    using CommInitRankFn = int (*)(void** comm, int nranks, NcclId id, int rank);
    using BroadcastFn = int (*)(const void* send, void* recv, size_t count, int datatype, int root, void* comm, cudaStream_t);
    using AllGatherFn = int (*)(const void* send, void* recv, size_t sendcount, int datatype, void* comm, cudaStream_t);
    using CommDestroyFn = int (*)(void* comm);
    using GetErrorStringFn = const char* (*)(int);

    struct NcclApi
    {
        void*            handle = nullptr;
        GetUniqueIdFn    get_unique_id = nullptr;
        CommInitRankFn   comm_init_rank = nullptr;
        BroadcastFn      broadcast = nullptr;
        AllGatherFn      all_gather = nullptr;
        CommDestroyFn    comm_destroy = nullptr;
        GetErrorStringFn error_string = nullptr;
        bool             ok = false;
        std::string      why; // why `ok` is false, for the error message
    };

    const NcclApi& nccl()
    {
        static NcclApi        api;
        static std::once_flag once;
        std::call_once(once, [] {
            void*       h        = nullptr;
            const char* override = std::getenv("B200WMMA_NCCL_LIBRARY");
            if(override && *override)
            {
                h = dlopen(override, RTLD_NOW | RTLD_GLOBAL);
                if(!h)
                {
                    api.why = std::string("B200WMMA_NCCL_LIBRARY=") + override + " cannot be opened";
                    return;
                }
            }
            else
            {
                h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD); // already in the process?
                if(!h)
                    h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
                if(!h)
                    h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
                if(!h)
                {
                    api.why = "libnccl.so.2 cannot be opened";
                    return;
                }
            }
            api.handle         = h;
            api.get_unique_id  = reinterpret_cast<GetUniqueIdFn>(dlsym(h, "ncclGetUniqueId"));
            api.comm_init_rank = reinterpret_cast<CommInitRankFn>(dlsym(h, "ncclCommInitRank"));
            api.broadcast      = reinterpret_cast<BroadcastFn>(dlsym(h, "ncclBroadcast"));
            api.all_gather     = reinterpret_cast<AllGatherFn>(dlsym(h, "ncclAllGather"));
            api.comm_destroy   = reinterpret_cast<CommDestroyFn>(dlsym(h, "ncclCommDestroy"));
            api.error_string   = reinterpret_cast<GetErrorStringFn>(dlsym(h, "ncclGetErrorString"));
            api.ok = api.get_unique_id && api.comm_init_rank && api.broadcast && api.all_gather && api.comm_destroy;
            if(!api.ok)
                api.why = "the NCCL library lacks one of ncclGetUniqueId / ncclCommInitRank / ncclBroadcast / ncclAllGather / "
                          "ncclCommDestroy";
        });
        return api;
    }

    const char* nccl_msg(int rc)
    {
        const NcclApi& n = nccl();
        return n.error_string ? n.error_string(rc) : "NCCL error";
    }
    constexpr int NCCL_INT8 = 0; // ncclInt8 / ncclChar
} // namespace

struct b200wmma_mg
{
    void* comm   = nullptr;
    int   rank   = 0;
    int   nranks = 0;
    int   device = 0;
};

extern "C" int b200wmma_mg_unique_id(void* id_out)
{
    using namespace b200wmma;
    clear_error();
    B200_REQUIRE(id_out, B200WMMA_ERR_INVALID_ARG, "mg_unique_id: id_out must be non-null");
    const NcclApi& n = nccl();
    B200_REQUIRE(n.ok, B200WMMA_ERR_UNSUPPORTED, "mg_unique_id: NCCL is not available (%s)", n.why.c_str());
    NcclId id;
    const int rc = n.get_unique_id(&id);
    B200_REQUIRE(rc == 0, B200WMMA_ERR_UNSUPPORTED, "mg_unique_id: ncclGetUniqueId failed: %s", nccl_msg(rc));
    std::memcpy(id_out, &id, sizeof(id));
    return B200WMMA_OK;
}

extern "C" int b200wmma_mg_create(b200wmma_mg** out, const void* id, int rank, int nranks)
{
    using namespace b200wmma;
    clear_error();
    B200_REQUIRE(out && id, B200WMMA_ERR_INVALID_ARG, "mg_create: out and id must be non-null");
    *out = nullptr;
    B200_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, B200WMMA_ERR_INVALID_ARG, "mg_create: bad rank %d of %d", rank,
                 nranks);
    const NcclApi& n = nccl();
    B200_REQUIRE(n.ok, B200WMMA_ERR_UNSUPPORTED, "mg_create: NCCL is not available (%s)", n.why.c_str());
    b200wmma_mg* mg = new(std::nothrow) b200wmma_mg();
    B200_REQUIRE(mg, B200WMMA_ERR_CUDA, "mg_create: out of host memory");
    cudaError_t e = cudaGetDevice(&mg->device);
    if(e != cudaSuccess)
    {
        delete mg;
        return set_error(B200WMMA_ERR_NO_DEVICE, "mg_create: no current CUDA device: %s", cudaGetErrorString(e));
    }
    NcclId nid;
    std::memcpy(&nid, id, sizeof(nid));
    const int rc = n.comm_init_rank(&mg->comm, nranks, nid, rank);
    if(rc != 0)
    {
        delete mg;
        return set_error(B200WMMA_ERR_UNSUPPORTED,
                         "mg_create: ncclCommInitRank failed (%s): no multi-GPU group; the single-GPU entry points still work",
                         nccl_msg(rc));
    }
    mg->rank   = rank;
    mg->nranks = nranks;
    // Warm the communicator: NCCL sets up its channels on the first collective of each kind, which would otherwise land
    // inside the first timed broadcast / gather.  One small broadcast and one small all-gather on a scratch buffer.
    if(nranks > 1)
    {
        void*        scratch = nullptr;
        const size_t per     = 4096;
        cudaError_t  ce      = cudaMalloc(&scratch, per * static_cast<size_t>(nranks));
        int          wrc     = 0;
        if(ce == cudaSuccess)
        {
            ce = cudaMemset(scratch, 0, per * static_cast<size_t>(nranks));
            if(ce == cudaSuccess)
                wrc = n.broadcast(scratch, scratch, per, NCCL_INT8, 0, mg->comm, nullptr);
            if(ce == cudaSuccess && wrc == 0)
                wrc = n.all_gather(static_cast<char*>(scratch) + per * static_cast<size_t>(rank), scratch, per, NCCL_INT8,
                                   mg->comm, nullptr);
            if(ce == cudaSuccess)
                ce = cudaStreamSynchronize(nullptr);
            cudaFree(scratch);
        }
        if(ce != cudaSuccess || wrc != 0)
        {
            n.comm_destroy(mg->comm);
            delete mg;
            return set_error(B200WMMA_ERR_UNSUPPORTED, "mg_create: the first collective on the new group failed (%s)",
                             ce != cudaSuccess ? cudaGetErrorString(ce) : nccl_msg(wrc));
        }
    }
    *out = mg;
    return B200WMMA_OK;
}

namespace b200wmma
{
    int mg_device(const b200wmma_mg* mg)
    {
        return mg ? mg->device : -1;
    }
    // The collectives without the device switch of the public entry points: the caller has made mg's device current.
    int mg_broadcast_here(b200wmma_mg* mg, void* buf, size_t bytes, int root, cudaStream_t stream)
    {
        const int rc = nccl().broadcast(buf, buf, bytes, NCCL_INT8, root, mg->comm, stream);
        B200_REQUIRE(rc == 0, B200WMMA_ERR_CUDA, "ncclBroadcast failed: %s", nccl_msg(rc));
        return B200WMMA_OK;
    }
    int mg_allgather_here(b200wmma_mg* mg, void* buf, size_t bytes_per_rank, cudaStream_t stream)
    {
        const int rc = nccl().all_gather(static_cast<char*>(buf) + bytes_per_rank * static_cast<size_t>(mg->rank), buf,
                                         bytes_per_rank, NCCL_INT8, mg->comm, stream);
        B200_REQUIRE(rc == 0, B200WMMA_ERR_CUDA, "ncclAllGather failed: %s", nccl_msg(rc));
        return B200WMMA_OK;
    }
} // namespace b200wmma

extern "C" int b200wmma_mg_broadcast(b200wmma_mg* mg, void* buf, size_t bytes, int root, void* stream)
{
    using namespace b200wmma;
    clear_error();
    B200_REQUIRE(mg && mg->comm, B200WMMA_ERR_INVALID_ARG, "mg_broadcast: mg must be a live handle");
    B200_REQUIRE(buf && bytes, B200WMMA_ERR_INVALID_ARG, "mg_broadcast: buf must be non-null and bytes non-zero");
    B200_REQUIRE(root >= 0 && root < mg->nranks, B200WMMA_ERR_INVALID_ARG, "mg_broadcast: bad root %d of %d", root, mg->nranks);
    B200_CHECK_CUDA(cudaSetDevice(mg->device));
    const int rc = nccl().broadcast(buf, buf, bytes, NCCL_INT8, root, mg->comm, static_cast<cudaStream_t>(stream));
    B200_REQUIRE(rc == 0, B200WMMA_ERR_CUDA, "ncclBroadcast failed: %s", nccl_msg(rc));
    return B200WMMA_OK;
}

extern "C" int b200wmma_mg_allgather(b200wmma_mg* mg, void* buf, size_t bytes_per_rank, void* stream)
{
    using namespace b200wmma;
    clear_error();
    B200_REQUIRE(mg && mg->comm, B200WMMA_ERR_INVALID_ARG, "mg_allgather: mg must be a live handle");
    B200_REQUIRE(buf && bytes_per_rank, B200WMMA_ERR_INVALID_ARG, "mg_allgather: buf must be non-null and bytes_per_rank non-zero");
    B200_CHECK_CUDA(cudaSetDevice(mg->device));
    return mg_allgather_here(mg, buf, bytes_per_rank, static_cast<cudaStream_t>(stream));
}

extern "C" int b200wmma_mg_destroy(b200wmma_mg* mg)
{
    using namespace b200wmma;
    clear_error();
    if(!mg)
        return B200WMMA_OK;
    int rc = 0;
    if(mg->comm)
    {
        cudaSetDevice(mg->device);
        rc = nccl().comm_destroy(mg->comm);
    }
    delete mg;
    B200_REQUIRE(rc == 0, B200WMMA_ERR_CUDA, "ncclCommDestroy failed: %s", nccl_msg(rc));
    return B200WMMA_OK;
}

extern "C" int b200wmma_mg_rank(const b200wmma_mg* mg)
{
    return mg ? mg->rank : -1;
}

extern "C" int b200wmma_mg_size(const b200wmma_mg* mg)
{
    return mg ? mg->nranks : 0;
}

// Contiguous, equally sized share [begin, begin + count) of `total` units for part `index` of `parts`; `total` must be
// a multiple of parts * granule (granule: the unit the kernels want whole, e.g. 16 columns).
extern "C" int b200wmma_shard_range(uint64_t total, uint32_t parts, uint32_t index, uint32_t granule, uint64_t* begin,
                                    uint64_t* count)
{
    using namespace b200wmma;
    clear_error();
    B200_REQUIRE(begin && count, B200WMMA_ERR_INVALID_ARG, "shard_range: begin and count must be non-null");
    B200_REQUIRE(parts >= 1 && index < parts && granule >= 1, B200WMMA_ERR_INVALID_ARG, "shard_range: bad part %u of %u", index,
                 parts);
    B200_REQUIRE(total % (static_cast<uint64_t>(parts) * granule) == 0, B200WMMA_ERR_UNSUPPORTED,
                 "shard_range: %llu units do not split into %u parts of whole granules of %u",
                 static_cast<unsigned long long>(total), parts, granule);
    *count = total / parts;
    *begin = *count * index;
    return B200WMMA_OK;
}
