// A CUDA backend of halo-flash's device interface (halo::rt::Device, src/rt/device.hpp:77-137) whose
// kernels are the sm_100a replacements of libhalo_b200.so. This is the file a maintainer adds next to
// src/rt/hip_device.cpp and src/rt/hrx_device.cpp: the engines (src/engine/*.cpp) contain no device code
// and call only this interface, so they drive the replacement kernels unchanged.
//
// It is compiled against the reference's own header (-I<reference>/src) and is not part of
// libhalo_b200.so, whose C ABI has no C++ types.
#ifndef HALO_B200_RT_CUDA_DEVICE_HPP_
#define HALO_B200_RT_CUDA_DEVICE_HPP_

#include <memory>
#include <string>

#include "rt/device.hpp"

namespace halo::rt {

// The value a maintainer would add to `enum class Backend` (src/rt/device.hpp:23).
inline constexpr Backend kBackendCuda = static_cast<Backend>(2);

// One device, one non-blocking stream (as HipDevice, src/rt/hip_device.cpp:49-50). Fails with a
// message when there is no CUDA device: there is no CPU fallback behind this interface.
std::unique_ptr<Device> CreateCudaDevice(int ordinal, std::string* error);

}  // namespace halo::rt

#endif  // HALO_B200_RT_CUDA_DEVICE_HPP_
