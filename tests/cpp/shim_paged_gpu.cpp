// The reference's free functions (src/machina/paged_attention.h:27-71) called from C++ exactly as
// src/machina/paged_attention.cu:353-367 and :616-619 call them, but through include/deusridet_shim.hpp and
// libdrkv.so, on a GPU: batched K/V write, single-token K/V write with the position on the device, decode
// attention.  Inputs and expected results come from a directory of raw files written by the Python test
// (a case recorded from the reference's own kernels); this program checks the pool bytes exactly and the
// attention output within max-abs 2e-3, and prints SHIM_GPU OK.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "deusridet_shim.hpp"

template <typename T>
static std::vector<T> slurp(const std::string& path) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    if (!f) {
        std::fprintf(stderr, "cannot read %s\n", path.c_str());
        std::exit(2);
    }
    const size_t bytes = (size_t)f.tellg();
    std::vector<T> v(bytes / sizeof(T));
    f.seekg(0);
    f.read(reinterpret_cast<char*>(v.data()), (std::streamsize)bytes);
    return v;
}

template <typename T>
static T* to_device(const std::vector<T>& v) {
    T* d = nullptr;
    if (cudaMalloc(&d, v.size() * sizeof(T) + 16) != cudaSuccess ||
        cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess) {
        std::fprintf(stderr, "device copy failed\n");
        std::exit(2);
    }
    return d;
}

int main(int argc, char** argv) {
    if (argc != 2) {
        std::fprintf(stderr, "usage: %s CASE_DIRECTORY\n", argv[0]);
        return 2;
    }
    const std::string dir = std::string(argv[1]) + "/";
    int hq, hkv, d, rot, page, layers, layer, seq_len, m_batch, max_pages;
    float theta;
    {
        std::ifstream meta(dir + "meta.txt");
        if (!(meta >> hq >> hkv >> d >> rot >> theta >> page >> layers >> layer >> seq_len >> m_batch >> max_pages)) {
            std::fprintf(stderr, "bad meta.txt\n");
            return 2;
        }
    }
    // what the reference reads from its ModelConfig statics (src/machina/paged_attention.cu:110-114)
    drkv_geometry& g = deusridet::shim_geometry();
    g = {layers, hq, hkv, d, page, DRKV_DTYPE_F16, rot, theta};

    auto pool = slurp<uint16_t>(dir + "pool.bin");
    auto table = slurp<int32_t>(dir + "table.bin");
    auto kb = slurp<uint16_t>(dir + "kb.bin"), vb = slurp<uint16_t>(dir + "vb.bin");
    auto k1 = slurp<uint16_t>(dir + "k1.bin"), v1 = slurp<uint16_t>(dir + "v1.bin");
    auto q = slurp<uint16_t>(dir + "q.bin");
    auto want_pool = slurp<uint16_t>(dir + "want_pool.bin"), want_out = slurp<uint16_t>(dir + "want_out.bin");

    __half* d_pool = reinterpret_cast<__half*>(to_device(pool));
    int* d_table = to_device(table);
    __half *d_kb = reinterpret_cast<__half*>(to_device(kb)), *d_vb = reinterpret_cast<__half*>(to_device(vb));
    __half *d_k1 = reinterpret_cast<__half*>(to_device(k1)), *d_v1 = reinterpret_cast<__half*>(to_device(v1));
    __half* d_q = reinterpret_cast<__half*>(to_device(q));
    std::vector<uint16_t> out(want_out.size(), 0);
    __half* d_out = reinterpret_cast<__half*>(to_device(out));
    cudaStream_t stream;
    cudaStreamCreate(&stream);

    int pos = seq_len;
    if (m_batch > 0) {
        deusridet::paged_kv_cache_write_batch(d_kb, d_vb, d_pool, d_table, layer, pos, m_batch, max_pages, page, stream);
        pos += m_batch;
    }
    std::vector<int32_t> h_pos(1, pos);
    int* d_pos = to_device(h_pos);
    deusridet::paged_kv_cache_write(d_k1, d_v1, d_pool, d_table, layer, d_pos, max_pages, page, stream);
    if (!deusridet::shim_reserve_decode_scratch(pos + 1, page)) {       // as a host would, before capturing its step
        std::fprintf(stderr, "scratch reservation failed\n");
        return 1;
    }
    deusridet::paged_gqa_decode_attention(d_q, d_pool, d_table, d_out, layer, pos + 1, max_pages, page,
                                          1.0f / std::sqrt((float)d), stream);
    if (!deusridet::shim_decode_kernels_ok(stream)) return 1;
    if (cudaStreamSynchronize(stream) != cudaSuccess) {
        std::fprintf(stderr, "stream failed: %s\n", cudaGetErrorString(cudaGetLastError()));
        return 1;
    }
    std::vector<uint16_t> got_pool(pool.size());
    cudaMemcpy(got_pool.data(), d_pool, pool.size() * 2, cudaMemcpyDeviceToHost);
    cudaMemcpy(out.data(), d_out, out.size() * 2, cudaMemcpyDeviceToHost);
    size_t bad = 0;
    for (size_t i = 0; i < pool.size(); i++) bad += got_pool[i] != want_pool[i];
    float worst = 0.f;
    for (size_t i = 0; i < out.size(); i++) {
        __half a, b;
        std::memcpy(&a, &out[i], 2);
        std::memcpy(&b, &want_out[i], 2);
        worst = std::fmax(worst, std::fabs(__half2float(a) - __half2float(b)));
    }
    std::printf("pool elements that differ: %zu, attention max-abs error: %g\n", bad, worst);
    if (bad != 0 || !(worst <= 2e-3f)) return 1;
    std::printf("SHIM_GPU OK\n");
    return 0;
}
