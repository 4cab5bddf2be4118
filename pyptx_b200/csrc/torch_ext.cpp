// pybind11 fast path for the PyTorch eager launch.
//
// Same two functions as the reference's extension (pyptx/_shim/torch_ext.cpp:14-80):
//   load_shim(path)      dlopen the C-ABI library and resolve its raw launch entry
//   launch_kernel(handle, stream, inputs, out_shapes, out_dtypes) -> outputs
// launch_kernel allocates the outputs with torch::empty on the first input's device, builds
// the void*[] of inputs then outputs and makes one call into pb200_launch_raw.  Unlike the
// reference, the error buffer is per call (no shared static buffer), and inputs are checked
// for device / contiguity before the call.
#include <torch/extension.h>

#include <dlfcn.h>

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

using LaunchRawFn = int (*)(int64_t, uint64_t, void**, size_t, char*);
LaunchRawFn g_launch_raw = nullptr;
void* g_lib = nullptr;

void load_shim(const std::string& path) {
    void* lib = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (!lib) throw std::runtime_error(std::string("pyptx_b200: dlopen failed: ") + dlerror());
    void* sym = dlsym(lib, "pb200_launch_raw");
    if (!sym) throw std::runtime_error("pyptx_b200: pb200_launch_raw not found in " + path);
    g_lib = lib;
    g_launch_raw = reinterpret_cast<LaunchRawFn>(sym);
}

std::vector<torch::Tensor> launch_kernel(int64_t handle, int64_t stream,
                                         const std::vector<torch::Tensor>& inputs,
                                         const std::vector<std::vector<int64_t>>& out_shapes,
                                         const std::vector<int64_t>& out_dtypes) {
    if (!g_launch_raw) throw std::runtime_error("pyptx_b200: load_shim() has not been called");
    if (inputs.empty()) throw std::invalid_argument("pyptx_b200: a kernel call requires at least one input");
    if (out_shapes.size() != out_dtypes.size()) throw std::invalid_argument("pyptx_b200: out_shapes / out_dtypes mismatch");
    const auto device = inputs[0].device();
    if (!device.is_cuda()) throw std::invalid_argument("pyptx_b200: inputs must be CUDA tensors (there is no CPU path)");
    std::vector<void*> ptrs;
    ptrs.reserve(inputs.size() + out_shapes.size());
    for (size_t i = 0; i < inputs.size(); ++i) {
        const auto& t = inputs[i];
        if (t.device() != device) throw std::invalid_argument("pyptx_b200: input " + std::to_string(i) + " is on another device");
        if (!t.is_contiguous()) throw std::invalid_argument("pyptx_b200: input " + std::to_string(i) + " is not contiguous");
        ptrs.push_back(t.data_ptr());
    }
    std::vector<torch::Tensor> outs;
    outs.reserve(out_shapes.size());
    for (size_t i = 0; i < out_shapes.size(); ++i) {
        auto opts = torch::TensorOptions().dtype(static_cast<c10::ScalarType>(out_dtypes[i])).device(device);
        outs.push_back(torch::empty(out_shapes[i], opts));
        ptrs.push_back(outs.back().data_ptr());
    }
    char err[128] = {0};
    int rc;
    {
        pybind11::gil_scoped_release nogil;
        rc = g_launch_raw(handle, static_cast<uint64_t>(stream), ptrs.data(), ptrs.size(), err);
    }
    if (rc != 0)
        throw std::runtime_error("pyptx_b200: pb200_launch_raw failed (code " + std::to_string(rc) + "): " + err);
    return outs;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("load_shim", &load_shim, "dlopen the C-ABI library");
    m.def("launch_kernel", &launch_kernel, "allocate outputs and launch a registered kernel");
}
