// HAL of the `c-b200` backend: the `namespace ab` interface the reference's runtime is written
// against (backends/c-rocm/include/backend.hpp:46-253, shared by c-cuda), on top of the antares_b200
// C ABI.  Including this header as `backend.hpp` lets the reference's unmodified
// graph_evaluator/execute_module.hpp and run_graph.cpp load, run, digest and time this library's
// kernels:
//
//   g++ <reference>/graph_evaluator/run_graph.cpp -std=c++17 -D__BACKEND__=\"c-b200\" \
//       -I include/c-b200 -I include -L antares_b200 -lantares_b200 -ldl -lpthread
//
//; eval_flags(c-b200): -lantares_b200
//
// Differences from the CUDA HAL it stands beside, all forced by there being no run-time compiler:
//   moduleCompile   returns the text unchanged (the reference shells out to nvcc, lines 116-159);
//   moduleLoad      hands the text to ab200_inject, which recognises the operator natively and
//                   binds it to a precompiled sm_100a kernel (the reference loads a fatbin, 161-170);
//   moduleGetFunction / launchKernel   carry the module key instead of a CUfunction; thread
//                   extents in the text are ignored (launch shapes belong to the kernels), and a
//                   launch is ab200_forward(key, pointers, stream) (reference: cuLaunchKernel, 199-219).
// Errors follow the reference's convention for a HAL (CHECK_OK prints and exits, line 8): this
// header is evaluator-side glue; the library underneath never exits.
#pragma once
#include <stdio.h>
#include <stdlib.h>

#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "antares_b200.h"

#if !defined(CHECK_OK)
#define CHECK_OK(x) ((x) ? 1 : (fprintf(stderr, "[CheckFail] %s:%d\n", __FILE__, __LINE__), exit(1), 0))
#endif

#define AB200_HAL_OK(call)                                                                   \
  do {                                                                                       \
    if ((call) != AB200_OK) {                                                                \
      fprintf(stderr, "[c-b200] %s failed: %s (%s:%d)\n", #call, ab200_last_error(), __FILE__, __LINE__); \
      exit(1);                                                                               \
    }                                                                                        \
  } while (0)

namespace ab {

static int _current_device = 0;
static std::unordered_map<size_t, std::vector<void *>> _free_list;  // released blocks by rounded size, reused before allocating

inline void init(int dev) {
  static bool done = false;
  if (dev < 0) {
    if (done) return;
    dev = 0;
  }
  _current_device = dev;
  AB200_HAL_OK(ab200_hal_set_device(dev));
  done = true;
}

inline void finalize() {}

inline size_t _round_size(size_t v) {  // next power of two below 1 GiB, exact above (the reference buckets the same way, lines 78-90)
  if (v >= ((size_t)1 << 30)) return v;
  size_t r = 1;
  while (r < v) r <<= 1;
  return r;
}

inline void *alloc(size_t byteSize, const std::vector<size_t> &shape, const std::string &dtype, const std::string &name) {
  init(-1);
  byteSize = _round_size(byteSize);
  auto &bucket = _free_list[byteSize];
  if (!bucket.empty()) {
    void *p = bucket.back();
    bucket.pop_back();
    return p;
  }
  void *p = (void *)1LU;  // zero-byte tensors get a non-null placeholder, as in the reference
  if (byteSize) AB200_HAL_OK(ab200_hal_malloc(&p, byteSize));
  return p;
}

inline void release(void *dptr, size_t byteSize) { _free_list[_round_size(byteSize)].push_back(dptr); }

inline std::string moduleCompile(const std::string &source) { return source; }

inline void *moduleLoad(const std::string &binary) {
  init(-1);
  int key = -1;
  AB200_HAL_OK(ab200_inject(binary.c_str(), &key));
  return (void *)(size_t)(key + 1);
}

inline std::vector<void *> moduleGetFunction(const void *hModule, const std::string &fname, const std::unordered_map<std::string, int> &threads) {
  return {const_cast<void *>(hModule)};
}

inline void launchKernel(std::vector<void *> &hFunc, const std::vector<void *> &krnl_args, void *stream) {
  const int key = (int)(size_t)hFunc[0] - 1;
  AB200_HAL_OK(ab200_forward(key, krnl_args.data(), (int)krnl_args.size(), stream));
}

inline void memcpyHtoD(void *dptr, void *hptr, size_t byteSize, void *stream) { AB200_HAL_OK(ab200_hal_memcpy(dptr, hptr, byteSize, 0, stream)); }
inline void memcpyDtoH(void *hptr, void *dptr, size_t byteSize, void *stream) { AB200_HAL_OK(ab200_hal_memcpy(hptr, dptr, byteSize, 1, stream)); }
inline void memcpyDtoD(void *dptr, void *dptr0, size_t byteSize, void *stream) { AB200_HAL_OK(ab200_hal_memcpy(dptr, dptr0, byteSize, 2, stream)); }

inline void synchronize(void *stream) { AB200_HAL_OK(ab200_hal_synchronize(stream)); }

inline void *recordTime(void *stream) {
  void *ev = nullptr;
  AB200_HAL_OK(ab200_hal_event_record(&ev, stream));
  return ev;
}

inline double convertToElapsedTime(void *hStart, void *hStop) {
  double sec = 0;
  AB200_HAL_OK(ab200_hal_event_elapsed(hStart, hStop, &sec));  // waits for the stop event, frees both
  return sec;
}

}  // namespace ab
