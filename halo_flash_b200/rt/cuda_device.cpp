// halo::rt::Device over the CUDA runtime and libhalo_b200.so. See cuda_device.hpp.
//
// Kernel(name) resolves a reference kernel name against halo_b200_kernel_name(); Launch() hands the
// reference's own grid, block and ordered rt::Arg list to halo_b200_launch(), which decodes row and
// batch counts from the grid exactly as the reference kernel reads blockIdx. Kernels outside the
// replaced path (GEMV / GEMM / attention / recurrence) are reported as absent by Kernel(), never
// emulated. LoadModule() accepts and ignores the gfx1151 code object: the replacement kernels are
// linked in.
#include "cuda_device.hpp"

#include <cuda_runtime.h>

#include <cstring>
#include <vector>

#include "halo_b200.h"

namespace halo::rt {
namespace {

bool Check(cudaError_t e, const char* what, std::string* error) {
  if (e == cudaSuccess) return true;
  if (error) *error = std::string(what) + ": " + cudaGetErrorString(e);
  return false;
}

// Makes a device current for the calling thread for the length of a scope. Every method below acts through the
// CUDA runtime, whose allocations, launches and memory queries go to the CURRENT device: a second Device object,
// or a worker thread that starts on device 0, must not send this object's work to another GPU.
class Current {
 public:
  explicit Current(int ordinal) : ordinal_(ordinal) {
    if (cudaGetDevice(&previous_) != cudaSuccess) previous_ = ordinal;
    if (previous_ != ordinal_) cudaSetDevice(ordinal_);
  }
  ~Current() {
    if (previous_ != ordinal_) cudaSetDevice(previous_);
  }
  Current(const Current&) = delete;
  Current& operator=(const Current&) = delete;

 private:
  int ordinal_, previous_ = 0;
};

class CudaDevice final : public Device {
 public:
  CudaDevice(int ordinal, cudaStream_t stream) : ordinal_(ordinal), stream_(stream) {}
  ~CudaDevice() override {
    const Current here(ordinal_);
    cudaStreamSynchronize(stream_);
    cudaStreamDestroy(stream_);
  }

  Backend backend() const noexcept override { return kBackendCuda; }

  Buffer Alloc(std::size_t bytes, std::string* error) override {
    const Current here(ordinal_);
    Buffer b;
    void* p = nullptr;
    if (!Check(cudaMalloc(&p, bytes ? bytes : 1), "cudaMalloc", error)) return b;
    b.device = p;
    b.bytes = bytes;
    return b;
  }
  void Free(Buffer& buffer) noexcept override {
    const Current here(ordinal_);
    if (buffer.device) cudaFree(buffer.device);
    buffer = {};
  }

  bool Upload(const Buffer& dst, std::size_t offset, const void* src, std::size_t bytes, std::string* error) override {
    const Current here(ordinal_);
    if (!InRange(dst, offset, bytes, "Upload", error) || !NotCapturing("Upload", error)) return false;
    if (!Check(cudaMemcpyAsync(static_cast<char*>(dst.device) + offset, src, bytes, cudaMemcpyHostToDevice, stream_),
               "Upload", error))
      return false;
    return Check(cudaStreamSynchronize(stream_), "Upload", error);
  }
  bool UploadAsync(const Buffer& dst, std::size_t offset, const void* src, std::size_t bytes,
                   std::string* error) override {
    const Current here(ordinal_);
    if (!InRange(dst, offset, bytes, "UploadAsync", error) || !NotCapturing("UploadAsync", error)) return false;
    return Check(cudaMemcpyAsync(static_cast<char*>(dst.device) + offset, src, bytes, cudaMemcpyHostToDevice, stream_),
                 "UploadAsync", error);
  }
  bool Download(const Buffer& src, std::size_t offset, void* dst, std::size_t bytes, std::string* error) override {
    const Current here(ordinal_);
    if (!InRange(src, offset, bytes, "Download", error) || !NotCapturing("Download", error)) return false;
    if (!Check(cudaMemcpyAsync(dst, static_cast<const char*>(src.device) + offset, bytes, cudaMemcpyDeviceToHost, stream_),
               "Download", error))
      return false;
    return Check(cudaStreamSynchronize(stream_), "Download", error);  // device faults surface here
  }
  bool Fill(const Buffer& dst, std::uint8_t value, std::string* error) override {
    const Current here(ordinal_);
    return Check(cudaMemsetAsync(dst.device, value, dst.bytes, stream_), "Fill", error);  // capturable
  }

  void* AllocHost(std::size_t bytes, std::string* error) override {
    const Current here(ordinal_);
    void* p = nullptr;
    if (!Check(cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault), "cudaHostAlloc", error)) return nullptr;
    return p;
  }
  void FreeHost(void* p) noexcept override {
    const Current here(ordinal_);
    if (p) cudaFreeHost(p);
  }
  std::size_t AvailableBytes() const override {
    const Current here(ordinal_);
    std::size_t free_b = 0, total = 0;
    return cudaMemGetInfo(&free_b, &total) == cudaSuccess ? free_b : SIZE_MAX;
  }

  bool LoadModule(std::span<const std::uint8_t>, std::string*) override { return true; }

  KernelId Kernel(std::string_view name, std::string* error) override {
    for (std::size_t i = 0; i < names_.size(); ++i)
      if (names_[i] == name) return static_cast<KernelId>(i);
    for (std::size_t i = 0; i < halo_b200_kernel_count(); ++i) {
      if (name == halo_b200_kernel_name(i)) {
        names_.emplace_back(name);
        return static_cast<KernelId>(names_.size() - 1);
      }
    }
    if (error) *error = "kernel " + std::string(name) + " is not part of the replaced elementwise path";
    return -1;
  }

  bool Launch(KernelId kernel, Dim3 grid, Dim3 block, std::span<const Arg> args, std::string* error) override {
    const Current here(ordinal_);
    if (kernel < 0 || static_cast<std::size_t>(kernel) >= names_.size()) {
      if (error) *error = "Launch: invalid kernel id";
      return false;
    }
    std::vector<halo_b200_arg> a(args.size());
    for (std::size_t i = 0; i < args.size(); ++i) {
      std::memset(&a[i], 0, sizeof(a[i]));
      if (args[i].kind == Arg::Kind::kBuffer) {
        a[i].is_buffer = 1;
        a[i].v.ptr = static_cast<char*>(args[i].buffer.device) + args[i].offset;
      } else {
        a[i].size = args[i].size;
        std::memcpy(a[i].v.bytes, args[i].bytes, args[i].size);
      }
    }
    const std::uint32_t g[3] = {grid.x, grid.y, grid.z}, b[3] = {block.x, block.y, block.z};
    char err[320];
    if (halo_b200_launch(stream_, names_[kernel].c_str(), a.data(), a.size(), g, b, err, sizeof err) == 0) return true;
    if (error) *error = err;  // launch errors are reported at the launch (src/engine/flash_next_gpu.cpp:149-152)
    return false;
  }

  bool Synchronize(std::string* error) override {
    const Current here(ordinal_);
    if (!NotCapturing("Synchronize", error)) return false;
    return Check(cudaStreamSynchronize(stream_), "Synchronize", error);
  }

  bool BeginCapture(std::string* error) override {
    const Current here(ordinal_);
    if (capturing_) {
      if (error) *error = "BeginCapture: already capturing";
      return false;
    }
    if (!Check(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal), "BeginCapture", error)) return false;
    capturing_ = true;
    return true;
  }
  bool EndCapture(Graph* out, std::string* error) override {
    const Current here(ordinal_);
    if (!capturing_) {
      if (error) *error = "EndCapture: not capturing";
      return false;
    }
    capturing_ = false;
    cudaGraph_t graph = nullptr;
    if (!Check(cudaStreamEndCapture(stream_, &graph), "EndCapture", error)) return false;
    cudaGraphExec_t exec = nullptr;
    const bool ok = Check(cudaGraphInstantiate(&exec, graph, 0), "cudaGraphInstantiate", error);
    cudaGraphDestroy(graph);
    if (!ok) return false;
    out->exec = exec;
    return true;
  }
  bool LaunchGraph(const Graph& graph, std::string* error) override {
    const Current here(ordinal_);
    if (!graph.exec) {
      if (error) *error = "LaunchGraph: empty graph";
      return false;
    }
    return Check(cudaGraphLaunch(static_cast<cudaGraphExec_t>(graph.exec), stream_), "LaunchGraph", error);
  }
  void FreeGraph(Graph& graph) noexcept override {
    const Current here(ordinal_);
    if (graph.exec) cudaGraphExecDestroy(static_cast<cudaGraphExec_t>(graph.exec));
    graph = {};
  }

 private:
  bool InRange(const Buffer& b, std::size_t offset, std::size_t bytes, const char* what, std::string* error) const {
    if (b.device && offset <= b.bytes && bytes <= b.bytes - offset) return true;
    if (error) *error = std::string(what) + ": range outside the buffer";
    return false;
  }
  bool NotCapturing(const char* what, std::string* error) const {
    if (!capturing_) return true;
    if (error) *error = std::string(what) + ": not allowed while capturing";  // src/rt/device.hpp:131-133
    return false;
  }

  int ordinal_;
  cudaStream_t stream_;
  bool capturing_ = false;
  std::vector<std::string> names_;  // KernelId -> reference kernel name
};

}  // namespace

std::unique_ptr<Device> CreateCudaDevice(int ordinal, std::string* error) {
  int count = 0;
  if (!Check(cudaGetDeviceCount(&count), "cudaGetDeviceCount", error)) return nullptr;
  if (ordinal < 0 || ordinal >= count) {
    if (error) *error = "no CUDA device " + std::to_string(ordinal);
    return nullptr;
  }
  if (!Check(cudaSetDevice(ordinal), "cudaSetDevice", error)) return nullptr;
  cudaStream_t stream = nullptr;
  if (!Check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate", error)) return nullptr;
  return std::make_unique<CudaDevice>(ordinal, stream);
}

}  // namespace halo::rt
