// C calling convention for the reference's own launchers, so tests can drive format37/kvskip's
// CUDA kernels (compiled for sm_100a from the reference checkout, see oracle/Makefile) side by
// side with this repository's library on the same GPU.  TEST INFRASTRUCTURE ONLY.
//
// The entry points take this repository's parameter blocks (include/kvskip_b200.h), which have
// the same field order and types as the reference's kvskip::Params / PlanParams / UpdateParams
// (kernels/kvskip.h:13-111); the static_asserts below keep that honest.
#include <cuda_runtime.h>

#include <exception>
#include <string>

#include "../include/kvskip_b200.h"
#include "kvskip.h"   // the reference's header, found through -I<reference>/kernels

static_assert(sizeof(kvskip_params) == sizeof(kvskip::Params), "attention parameter block differs");
static_assert(sizeof(kvskip_plan_params) == sizeof(kvskip::PlanParams), "plan parameter block differs");
static_assert(sizeof(kvskip_update_params) == sizeof(kvskip::UpdateParams), "update parameter block differs");
static_assert(offsetof(kvskip_params, lse_prev) == offsetof(kvskip::Params, lse_prev), "layout");
static_assert(offsetof(kvskip_params, blk_max) == offsetof(kvskip::Params, blk_max), "layout");
static_assert(offsetof(kvskip_plan_params, delta) == offsetof(kvskip::PlanParams, delta), "layout");
static_assert(offsetof(kvskip_update_params, level) == offsetof(kvskip::UpdateParams, level), "layout");

namespace {
thread_local std::string t_err;
template <typename F>
int guarded(F&& f) {
  try {
    f();
  } catch (const std::exception& e) {
    t_err = e.what();
    return -1;
  }
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    t_err = cudaGetErrorString(e);
    return -2;
  }
  return 0;
}
}  // namespace

extern "C" {
const char* kvref_last_error(void) { return t_err.c_str(); }

int kvref_launch_decode(const kvskip_params* p, int D, int G, int stages, int masked, int stats, int load_v,
                        void* stream) {
  return guarded([&] {
    kvskip::launch_decode(*reinterpret_cast<const kvskip::Params*>(p), D, G, stages, masked, stats, load_v,
                          static_cast<cudaStream_t>(stream));
  });
}
int kvref_launch_vskip1(const kvskip_params* p, int D, int G, void* stream) {
  return guarded([&] {
    kvskip::launch_vskip1(*reinterpret_cast<const kvskip::Params*>(p), D, G, static_cast<cudaStream_t>(stream));
  });
}
int kvref_launch_pv(const kvskip_params* p, int D, int G, void* stream) {
  return guarded([&] {
    kvskip::launch_pv(*reinterpret_cast<const kvskip::Params*>(p), D, G, static_cast<cudaStream_t>(stream));
  });
}
int kvref_launch_plan(const kvskip_plan_params* p, void* stream) {
  return guarded([&] {
    kvskip::launch_plan(*reinterpret_cast<const kvskip::PlanParams*>(p), static_cast<cudaStream_t>(stream));
  });
}
int kvref_launch_update(const kvskip_update_params* p, void* stream) {
  return guarded([&] {
    kvskip::launch_update(*reinterpret_cast<const kvskip::UpdateParams*>(p), static_cast<cudaStream_t>(stream));
  });
}
int kvref_launch_read(const void* x, int64_t bytes, uint32_t* out, int blocks, void* stream) {
  return guarded([&] { kvskip::launch_read(x, bytes, out, blocks, static_cast<cudaStream_t>(stream)); });
}
}
