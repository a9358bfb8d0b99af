// Test infrastructure, not product code.
//
// One translation unit of the reference's own native extension
// (csrc/attention/cuda/sm120/*.cu, built unchanged from where the reference tree lies),
// compiled for sm_100a so that its kernels can run on a B200 and pin the CPU oracle.
// The source to build is named on the command line: -DANEMOI_REF_SOURCE="<path>".
//
// The reference's host functions refuse every device but SM120
// (q128_microscaling_preparation.cu:1234-1238, h3_draft_probability.cu:576-586,
// h3_route_precision.cu:30-33).  Its kernels for preparation, routing and the FP16 / INT8
// cells use nothing that sm_100a lacks, so this wrapper answers the capability question
// with "12.0" and leaves everything else to the reference's code: same launchers, same
// grids, same kernels, same compiler flags.  The NVFP4 attention phase cannot be built this
// way (its block-scaled mma.sync does not assemble for sm_100a).
#include <cassert>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

namespace at::cuda {
inline const cudaDeviceProp* anemoi_ref_properties_as_sm120(c10::DeviceIndex device) {
  static thread_local cudaDeviceProp reported;
  reported = *getDeviceProperties(device);
  reported.major = 12;
  reported.minor = 0;
  return &reported;
}
}  // namespace at::cuda

#define getDeviceProperties anemoi_ref_properties_as_sm120
#define MPA_ROUTE_DEVICE_OK(properties) (true)

#include ANEMOI_REF_SOURCE
