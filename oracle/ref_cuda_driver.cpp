// TEST INFRASTRUCTURE — NOT THE PRODUCT.
//
// A C++ caller of the reference's own linalg API, linked from the reference's unmodified
// src/linalg/gemm_dispatch.cpp and src/linalg/gemm_cpu.cpp plus this repository's
// reference_shim/linalg_cuda_shim.cpp with -DT81LIB_USE_CUDA=1 (oracle/Makefile, target ref_cuda).
// It proves that the shim fills the reference's CUDA backend slot: the calls below are the
// reference's public entry points (include/t81/linalg/gemm.hpp:68-77,
// include/t81/linalg/gemm_gpu.hpp:82-118,162-214) and reach libt81_b200.so through the dispatcher.
//
//   ref_cuda_driver <mode> <input file> <output file>
// Input and output are raw little-endian arrays; tests/test_reference_shim.py writes the input,
// runs this program on a GPU and compares the output with the CPU oracle.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <span>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include <t81/linalg/gemm.hpp>
#include <t81/linalg/gemm_gpu.hpp>

#include "../t81lib_b200/reference_shim/t81_b200_linalg.hpp"

using t81::DeviceType;
using t81::ScalarType;
using t81::TensorMetadata;
using t81::core::limb;
namespace linalg = t81::linalg;

namespace {

struct Reader {
    FILE *f;
    template <typename T> std::vector<T> take(std::size_t n) {
        std::vector<T> v(n);
        if (n && std::fread(static_cast<void *>(v.data()), sizeof(T), n, f) != n) throw std::runtime_error("short input file");
        return v;
    }
    template <typename T> T one() { return take<T>(1)[0]; }
};

struct Writer {
    FILE *f;
    template <typename T> void put(const std::vector<T> &v) { if (!v.empty()) std::fwrite(v.data(), sizeof(T), v.size(), f); }
};

void cuda_ok(cudaError_t e, const char *what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// A device copy of a host array, described the way python/bindings.cpp:297-326 describes a torch CUDA tensor.
struct DeviceArray {
    void *ptr = nullptr;
    std::size_t bytes = 0;
    DeviceArray(const void *host, std::size_t n) : bytes(n) {
        cuda_ok(cudaMalloc(&ptr, n ? n : 16), "cudaMalloc");
        if (n) cuda_ok(cudaMemcpy(ptr, host, n, cudaMemcpyHostToDevice), "cudaMemcpy");
    }
    ~DeviceArray() { cudaFree(ptr); }
    template <typename T> std::vector<T> back() const {
        std::vector<T> v(bytes / sizeof(T));
        if (bytes) cuda_ok(cudaMemcpy(static_cast<void *>(v.data()), ptr, bytes, cudaMemcpyDeviceToHost), "cudaMemcpy");
        return v;
    }
};

TensorMetadata meta2d(void *ptr, ScalarType dtype, int64_t rows, int64_t cols, bool on_device) {
    TensorMetadata m;
    m.device_type = on_device ? DeviceType::CUDA : DeviceType::CPU;
    m.data_ptr = ptr;
    m.dtype = dtype;
    m.sizes = {rows, cols};
    m.strides = {cols, 1};
    m.requires_sync = on_device;
    return m;
}

TensorMetadata meta1d(void *ptr, int64_t n, bool on_device) {
    TensorMetadata m = t81::make_contiguous_metadata(static_cast<std::size_t>(n), ptr);
    m.device_type = on_device ? DeviceType::CUDA : DeviceType::CPU;
    m.requires_sync = on_device;
    return m;
}

// LIMB mode through every form of the reference API; writes five copies of C.
void run_limb(Reader in, Writer out) {
    const int M = in.one<int32_t>(), N = in.one<int32_t>(), KL = in.one<int32_t>();
    const float alpha = in.one<float>(), beta = in.one<float>();
    auto a = in.take<limb>((std::size_t)M * KL);
    auto b = in.take<limb>((std::size_t)KL * N);
    const auto c0 = in.take<float>((std::size_t)M * N);
    const int K = KL * limb::TRITS;

    auto c = c0;  // 1: span API, backend chosen by the reference (Auto -> CUDA when a device is present)
    linalg::gemm_ternary(a, b, c, M, N, K, alpha, beta);
    out.put(c);
    c = c0;       // 2: dispatcher with Backend::CUDA named explicitly
    linalg::detail::gemm_ternary_dispatch(a, b, c, M, N, K, alpha, beta, linalg::Backend::CUDA);
    out.put(c);
    c = c0;       // 3: the reference's own CPU kernel, for comparison in the same process
    linalg::detail::gemm_ternary_dispatch(a, b, c, M, N, K, alpha, beta, linalg::Backend::CPU);
    out.put(c);
    c = c0;       // 4: TensorMetadata over host arrays
    {
        TensorMetadata ma = meta2d(a.data(), ScalarType::TernaryLimb, M, KL, false);
        TensorMetadata mb = meta2d(b.data(), ScalarType::TernaryLimb, KL, N, false);
        TensorMetadata mc = meta2d(c.data(), ScalarType::Float, M, N, false);
        linalg::detail::gemm_ternary(ma, mb, mc, alpha, beta, linalg::Backend::Auto);
    }
    out.put(c);
    {             // 5: TensorMetadata over device memory (device_type CUDA, requires_sync)
        DeviceArray da(a.data(), a.size() * sizeof(limb)), db(b.data(), b.size() * sizeof(limb)), dc(c0.data(), c0.size() * 4);
        TensorMetadata ma = meta2d(da.ptr, ScalarType::TernaryLimb, M, KL, true);
        TensorMetadata mb = meta2d(db.ptr, ScalarType::TernaryLimb, KL, N, true);
        TensorMetadata mc = meta2d(dc.ptr, ScalarType::Float, M, N, true);
        linalg::detail::gemm_ternary(ma, mb, mc, alpha, beta, linalg::Backend::Auto);
        out.put(dc.back<float>());
    }
}

// TRIT mode (the additive overloads); writes three copies of C.
void run_trit(Reader in, Writer out) {
    const int M = in.one<int32_t>(), N = in.one<int32_t>(), KL = in.one<int32_t>();
    const float alpha = in.one<float>(), beta = in.one<float>();
    const int K = KL * limb::TRITS;
    auto a = in.take<limb>((std::size_t)M * KL);
    auto b = in.take<float>((std::size_t)K * N);
    const auto c0 = in.take<float>((std::size_t)M * N);

    auto c = c0;  // 1: span overload
    linalg::gemm_ternary(std::span<const limb>(a), std::span<const float>(b), std::span<float>(c), M, N, K, alpha, beta);
    out.put(c);
    c = c0;       // 2: TensorMetadata over host arrays
    {
        TensorMetadata ma = meta2d(a.data(), ScalarType::TernaryLimb, M, KL, false);
        TensorMetadata mb = meta2d(b.data(), ScalarType::Float, K, N, false);
        TensorMetadata mc = meta2d(c.data(), ScalarType::Float, M, N, false);
        linalg::detail::gemm_ternary_dense(ma, mb, mc, alpha, beta);
    }
    out.put(c);
    {             // 3: TensorMetadata over device memory
        DeviceArray da(a.data(), a.size() * sizeof(limb)), db(b.data(), b.size() * 4), dc(c0.data(), c0.size() * 4);
        TensorMetadata ma = meta2d(da.ptr, ScalarType::TernaryLimb, M, KL, true);
        TensorMetadata mb = meta2d(db.ptr, ScalarType::Float, K, N, true);
        TensorMetadata mc = meta2d(dc.ptr, ScalarType::Float, M, N, true);
        linalg::detail::gemm_ternary_dense(ma, mb, mc, alpha, beta);
        out.put(dc.back<float>());
    }
}

// where / clamp / lerp / addcmul with Backend::Auto, host arrays then device arrays: 8 result arrays.
void run_elementwise(Reader in, Writer out) {
    const int64_t n = in.one<int64_t>();
    const float lo = in.one<float>(), hi = in.one<float>(), value = in.one<float>();
    auto a = in.take<float>((std::size_t)n), b = in.take<float>((std::size_t)n), c = in.take<float>((std::size_t)n);
    for (int on_device = 0; on_device < 2; ++on_device) {
        DeviceArray da(a.data(), a.size() * 4), db(b.data(), b.size() * 4), dc(c.data(), c.size() * 4);
        for (int op = 0; op < 4; ++op) {
            std::vector<float> r((std::size_t)n, -7.0f);
            DeviceArray dr(r.data(), r.size() * 4);
            TensorMetadata ma = meta1d(on_device ? da.ptr : a.data(), n, on_device);
            TensorMetadata mb = meta1d(on_device ? db.ptr : b.data(), n, on_device);
            TensorMetadata mc = meta1d(on_device ? dc.ptr : c.data(), n, on_device);
            TensorMetadata mr = meta1d(on_device ? dr.ptr : r.data(), n, on_device);
            switch (op) {
                case 0: linalg::detail::where(ma, mb, mc, mr); break;
                case 1: linalg::detail::clamp(ma, mr, lo, hi); break;
                case 2: linalg::detail::lerp(ma, mb, mc, mr); break;
                default: linalg::detail::addcmul(ma, mb, mc, value, mr); break;
            }
            out.put(on_device ? dr.back<float>() : r);
        }
    }
}

// The exceptions the boundary raises; one line per case: "<case> <exception type> <message>".
void run_errors(Writer out) {
    std::string text;
    auto attempt = [&](const char *name, auto &&fn) {
        try {
            fn();
            text += std::string(name) + " none\n";
        } catch (const std::invalid_argument &e) {
            text += std::string(name) + " invalid_argument " + e.what() + "\n";
        } catch (const std::runtime_error &e) {
            text += std::string(name) + " runtime_error " + e.what() + "\n";
        }
    };
    std::vector<limb> a(2), b(2);
    std::vector<float> c(4, 1.0f), bf(96 * 2);
    attempt("negative", [&] { linalg::gemm_ternary(a, b, c, -1, 2, 48, 1.0f, 0.0f); });
    attempt("k_not_48", [&] { linalg::gemm_ternary(a, b, c, 2, 2, 47, 1.0f, 0.0f); });
    attempt("a_size", [&] { linalg::gemm_ternary(std::span<const limb>(a.data(), 1), b, c, 2, 2, 48, 1.0f, 0.0f); });
    attempt("empty", [&] { linalg::gemm_ternary(std::span<const limb>(), std::span<const limb>(), std::span<float>(), 0, 0, 0, 1.0f, 0.0f); });
    attempt("dense_b_size", [&] { linalg::gemm_ternary(std::span<const limb>(a), std::span<const float>(bf.data(), 5), std::span<float>(c), 2, 2, 48, 1.0f, 0.0f); });
    attempt("clamp_dtype", [&] {
        TensorMetadata in = meta1d(c.data(), 4, false), o = meta1d(c.data(), 4, false);
        in.dtype = ScalarType::Half;
        linalg::detail::clamp(in, o, 0.0f, 1.0f);
    });
    attempt("where_length", [&] {
        std::vector<float> s(3);
        TensorMetadata cond = meta1d(c.data(), 4, false), x = meta1d(s.data(), 3, false), y = meta1d(c.data(), 4, false), o = meta1d(c.data(), 4, false);
        linalg::detail::where(cond, x, y, o);
    });
    std::fwrite(text.data(), 1, text.size(), out.f);
}

}  // namespace

int main(int argc, char **argv) {
    if (argc != 4) {
        std::fprintf(stderr, "usage: %s limb|trit|elementwise|errors <input> <output>\n", argv[0]);
        return 2;
    }
    try {
        const std::string mode = argv[1];
        FILE *fi = std::fopen(argv[2], "rb"), *fo = std::fopen(argv[3], "wb");
        if (!fi || !fo) throw std::runtime_error("cannot open the input or output file");
        if (!linalg::detail::cuda_available()) throw std::runtime_error("no CUDA device: the reference would select its CPU backend");
        Reader in{fi};
        Writer out{fo};
        if (mode == "limb") run_limb(in, out);
        else if (mode == "trit") run_trit(in, out);
        else if (mode == "elementwise") run_elementwise(in, out);
        else if (mode == "errors") run_errors(out);
        else throw std::runtime_error("unknown mode " + mode);
        std::fclose(fi);
        std::fclose(fo);
    } catch (const std::exception &e) {
        std::fprintf(stderr, "ref_cuda_driver: %s\n", e.what());
        return 1;
    }
    return 0;
}
