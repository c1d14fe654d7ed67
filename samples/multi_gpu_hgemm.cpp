// Column-sharded fp16 GEMM on several GPUs from a C++ host, one process per GPU, on the C ABI's own plumbing
// (b200wmma_mg_*, b200wmma_shard_range).  The reference has no multi-GPU sample; the GEMM is the perf_hgemm form
// (samples/perf_hgemm.cpp:713-941: A row-major, B column-major, C / D row-major fp16, alpha = beta = 1).
//
// Usage: multi_gpu_hgemm <rank> <nranks> <id file> [m n k [run tag]]      (default 2048 x 4096 x 1024)
// Start one process per rank, all with the same id file path on a file system they share.  Rank r uses device r.
// Rank 0 creates the NCCL id and publishes it through the file; the others wait for it (30 s at most).  The file
// holds the run tag (any string, the same for all ranks of one run; give a fresh one per run, e.g. the launcher's pid)
// in front of the id, and readers ignore a file with another tag: an id left behind by an aborted run is never taken
// for this run's.  Rank 0 removes a stale file before it creates the id.
#include "common.hpp"

#include <chrono>
#include <cstring>
#include <string>
#include <thread>

constexpr size_t TAG_BYTES = 32;
static void      tag_field(const char* tag, char (&out)[TAG_BYTES])
{
    std::memset(out, 0, TAG_BYTES);
    std::strncpy(out, tag, TAG_BYTES - 1);
}

static bool publish_id(const char* path, const char* tag, const unsigned char* id)
{
    const std::string tmp = std::string(path) + ".tmp";
    FILE*             f   = std::fopen(tmp.c_str(), "wb");
    if(!f)
        return false;
    char field[TAG_BYTES];
    tag_field(tag, field);
    const bool ok = std::fwrite(field, 1, TAG_BYTES, f) == TAG_BYTES
                    && std::fwrite(id, 1, B200WMMA_MG_ID_BYTES, f) == B200WMMA_MG_ID_BYTES;
    std::fclose(f);
    return ok && std::rename(tmp.c_str(), path) == 0; // rename: readers never see a partial file
}

static bool fetch_id(const char* path, const char* tag, unsigned char* id)
{
    char want[TAG_BYTES], have[TAG_BYTES];
    tag_field(tag, want);
    for(int tries = 0; tries < 300; ++tries)
    {
        if(FILE* f = std::fopen(path, "rb"))
        {
            const bool got = std::fread(have, 1, TAG_BYTES, f) == TAG_BYTES
                             && std::fread(id, 1, B200WMMA_MG_ID_BYTES, f) == B200WMMA_MG_ID_BYTES;
            std::fclose(f);
            if(got && std::memcmp(want, have, TAG_BYTES) == 0)
                return true; // (a file with another run's tag is a leftover: keep waiting for this run's)
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(100));
    }
    return false;
}

int main(int argc, char** argv)
{
    if(argc < 4)
    {
        std::printf("usage: multi_gpu_hgemm <rank> <nranks> <id file> [m n k]\n");
        return 2;
    }
    const int      rank = std::atoi(argv[1]), nranks = std::atoi(argv[2]);
    const char*    id_path = argv[3];
    const uint32_t m = argc > 6 ? std::atoi(argv[4]) : 2048, n = argc > 6 ? std::atoi(argv[5]) : 4096,
                   k = argc > 6 ? std::atoi(argv[6]) : 1024;
    const char* run_tag = argc > 7 ? argv[7] : "untagged";
    CHECK_CUDA(cudaSetDevice(rank));

    unsigned char id[B200WMMA_MG_ID_BYTES];
    if(rank == 0)
    {
        std::remove(id_path); // whatever an earlier run left there
        CHECK_B200(b200wmma_mg_unique_id(id));
        if(!publish_id(id_path, run_tag, id))
        {
            std::printf("cannot write %s\n", id_path);
            return 1;
        }
    }
    else if(!fetch_id(id_path, run_tag, id))
    {
        std::printf("rank %d: no id in %s after 30 s\n", rank, id_path);
        return 1;
    }
    b200wmma_mg* mg = nullptr;
    CHECK_B200(b200wmma_mg_create(&mg, id, rank, nranks));

    uint64_t col0 = 0, ncols = 0;
    CHECK_B200(b200wmma_shard_range(n, nranks, rank, 16, &col0, &ncols));
    const uint32_t nl = static_cast<uint32_t>(ncols);

    // every rank could generate A; to exercise the broadcast only rank 0 does, the others start from zeros
    std::vector<__half> a(size_t(m) * k), b(size_t(nl) * k), c(size_t(m) * nl), d(size_t(m) * nl);
    for(size_t i = 0; i < a.size(); ++i)
        a[i] = __float2half(rank == 0 ? float(sample::uniform(1, i)) : 0.0f);
    for(uint32_t j = 0; j < nl; ++j) // this rank's columns of the column-major B: rows of B^T
        for(uint32_t h = 0; h < k; ++h)
            b[size_t(j) * k + h] = __float2half(float(sample::uniform(2, size_t(col0 + j) * k + h)));
    for(uint32_t i = 0; i < m; ++i)
        for(uint32_t j = 0; j < nl; ++j)
            c[size_t(i) * nl + j] = __float2half(float(sample::uniform(3, size_t(i) * n + col0 + j)));
    __half *da = sample::to_device(a), *db = sample::to_device(b), *dc = sample::to_device(c), *dd = nullptr;
    CHECK_CUDA(cudaMalloc(&dd, d.size() * sizeof(__half)));
    CHECK_CUDA(cudaMemset(dd, 0xFF, d.size() * sizeof(__half)));

    CHECK_B200(b200wmma_mg_broadcast(mg, da, a.size() * sizeof(__half), 0, nullptr)); // A is needed whole by every rank
    CHECK_CUDA(cudaDeviceSynchronize());
    const float ms = sample::time_launches(
        [&] {
            CHECK_B200(b200wmma_gemm_f16(m, nl, k, da, db, dc, dd, k, k, nl, nl, 1.0f, 1.0f, B200WMMA_ROW_MAJOR,
                                         B200WMMA_COL_MAJOR, B200WMMA_ROW_MAJOR, B200WMMA_OUT_F16, nullptr));
        },
        3, 10);
    std::printf("rank %d of %d: columns [%llu, %llu), %.4f ms, %.2f TFlops/s on this GPU\n", rank, nranks,
                static_cast<unsigned long long>(col0), static_cast<unsigned long long>(col0 + ncols), ms,
                sample::tflops(m, nl, k, ms));
    CHECK_CUDA(cudaMemcpy(d.data(), dd, d.size() * sizeof(__half), cudaMemcpyDeviceToHost));

    // check sampled rows of this rank's block against a double-precision dot product of the generated values
    double max_err = 0.0;
    for(uint32_t s = 0; s < 8; ++s)
    {
        const uint32_t i = (s == 7) ? m - 1 : uint32_t(sample::mix(43, s) % m);
        for(uint32_t j = 0; j < nl; ++j)
        {
            double acc = 0.0, mag = 0.0;
            for(uint32_t h = 0; h < k; ++h)
            {
                const double av = __half2float(__float2half(float(sample::uniform(1, size_t(i) * k + h))));
                const double bv = __half2float(b[size_t(j) * k + h]);
                acc += av * bv;
                mag += std::fabs(av * bv);
            }
            const double cv = __half2float(c[size_t(i) * nl + j]), ref = acc + cv;
            max_err = std::fmax(max_err, std::fabs(__half2float(d[size_t(i) * nl + j]) - ref) / std::fmax(mag + std::fabs(cv), 1e-30));
        }
    }
    CHECK_CUDA(cudaFree(da)); CHECK_CUDA(cudaFree(db)); CHECK_CUDA(cudaFree(dc)); CHECK_CUDA(cudaFree(dd));
    CHECK_B200(b200wmma_mg_destroy(mg));
    if(rank == 0)
        std::remove(id_path);
    return sample::report("multi_gpu_hgemm", max_err, 2e-3);
}
