// Shared definitions for the RBF attention kernels: tile geometry, argument blocks, status codes.
#pragma once

#include "ptx.cuh"

namespace rbf {

static constexpr int kTile = 128;       // rows of a query tile == keys of a key tile
static constexpr float kLog2e = 1.4426950408889634f;

// Status codes returned through the C ABI (0 = success).
enum Status : int {
  kOk = 0,
  kErrBadArgument = 1,     // null pointer, non-positive size, unsupported D / dtype
  kErrBadLayout = 2,       // stride or alignment the TMA engine cannot address
  kErrWorkspace = 3,       // workspace missing or too small
  kErrTensorMap = 4,       // cuTensorMapEncodeTiled failed or is unavailable
  kErrLaunch = 5,          // CUDA launch error
  kErrDevice = 6,          // a device-side bounded wait ran out (see rbf_b200_read_device_status)
};

// Number of key/query rows after padding to whole tiles; the per-row fp32 side arrays
// (key norms, query norms, delta) use this as their row pitch so that every tile read is in bounds.
__host__ __device__ inline int padded_rows(int n) { return (n + kTile - 1) / kTile * kTile; }

}  // namespace rbf
