// Stand-alone C++ runner for an AOTInductor package that contains a TensorProduct of this library.
//
//   run_package <liboeq_b200_torch.so> <package.pt2> <batch> <L1_dim> <L2_dim> <weight_numel>
//
// It loads the operator library (which registers libtorch_tp_jit::jit_* from C++), loads the package, runs it on
// inputs that the calling test can rebuild exactly (sines of an index ramp) and prints two checksums of the output.
// Counterpart of the reference's extension/test/load_aoti.cpp:16-62 (which compares with an e3nn package instead).
#include <ATen/ATen.h>
#include <c10/core/InferenceMode.h>
#include <dlfcn.h>
#include <torch/csrc/inductor/aoti_package/model_package_loader.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

static at::Tensor ramp(int64_t rows, int64_t cols, double scale) {
    return at::sin(at::arange(rows * cols, at::TensorOptions().dtype(at::kFloat).device(at::kCUDA)) * scale).reshape({rows, cols});
}

int main(int argc, const char* argv[]) {
    if (argc != 7) {
        std::fprintf(stderr, "usage: run_package <ops library> <package> <batch> <L1_dim> <L2_dim> <weight_numel>\n");
        return 2;
    }
    if (!dlopen(argv[1], RTLD_NOW | RTLD_GLOBAL)) {
        std::fprintf(stderr, "cannot load %s: %s\n", argv[1], dlerror());
        return 3;
    }
    const int64_t B = std::atoll(argv[3]), L1 = std::atoll(argv[4]), L2 = std::atoll(argv[5]), wn = std::atoll(argv[6]);
    c10::InferenceMode mode;
    try {
        std::vector<at::Tensor> inputs = {ramp(B, L1, 0.37), ramp(B, L2, 0.11), ramp(B, wn, 0.23)};
        torch::inductor::AOTIModelPackageLoader package(argv[2]);
        std::vector<at::Tensor> out = package.run(inputs);
        if (out.empty()) { std::fprintf(stderr, "the package returned nothing\n"); return 4; }
        const at::Tensor z = out[0].to(at::kDouble).cpu();
        std::printf("shape %lld %lld\nsum %.10e\nabs %.10e\n", (long long)z.size(0), (long long)z.size(1),
                    z.sum().item<double>(), z.abs().sum().item<double>());
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
    return 0;
}
