// TEST INFRASTRUCTURE ONLY: C-ABI doorway into the reference's own CPU runtime.
//
// This translation unit is the only code of ours in oracle/_ref/libantares_ref_mcpu.so.
// It #includes, from where they lie in the reference checkout,
//   graph_evaluator/execute_module.hpp      (ExecutionModule: header parse, kernel chain)
//   backends/c-mcpu/include/backend.hpp     (namespace ab: g++ JIT, dlopen, pinned thread pool)
// unmodified, exactly as the reference's evaluator (graph_evaluator/run_graph.cpp:6) and
// torch binding (frameworks/pytorch/main_ops.cc:9) do, and exposes create/compute/time so
// that Python (ctypes) can run kernel-source texts on it.  The reference's code generator
// needs a patched TVM that is not available offline, so the kernel-source texts are
// written by hand (oracle/ref_kernels.py) in the c-mcpu dialect that
// backends/c-scpu/config.py:22-49 emits.
//
// Not thread-safe (the reference runtime keeps thread_local/static state): call from one thread.
#include <string>
#include <vector>
#include <memory>
#include <chrono>
#include <unistd.h>

#include "execute_module.hpp"

namespace {
std::vector<std::unique_ptr<ExecutionModule>> g_modules;
}

extern "C" {

// Builds an ExecutionModule from kernel-source text (graph_evaluator/execute_module.hpp:274-319).
// The reference JIT writes its temporaries relative to the working directory, so the call
// runs inside `workdir`.  Returns a handle >= 0.
int ref_module_create(const char *source, const char *workdir) {
  char cwd[4096];
  if (!getcwd(cwd, sizeof(cwd))) return -1;
  if (workdir && *workdir && chdir(workdir) != 0) return -2;
  int handle = -3;
  try {
    g_modules.emplace_back(std::make_unique<ExecutionModule>(std::string(source), 0));
    handle = (int)g_modules.size() - 1;
  } catch (const std::exception &e) {
    fprintf(stderr, "[ref_shim] %s\n", e.what());
  }
  if (chdir(cwd) != 0) return -4;
  return handle;
}

int ref_module_num_inputs(int h) { return (int)g_modules[h]->global_inputs.size(); }
int ref_module_num_outputs(int h) { return (int)g_modules[h]->global_outputs.size(); }

// args = input pointers (sorted as in `// GLOBALS:`) followed by output pointers, the
// argument convention of frameworks/pytorch/main_ops.cc:36-44.
int ref_module_compute(int h, void **args) {
  g_modules[h]->compute(args);
  ab::synchronize(nullptr);
  return 0;
}

// Seconds per run by the evaluator's protocol (graph_evaluator/run_graph.cpp:214-236):
// one run; if it took under 2 s, min(1e4, 1/tpr) further runs (capped by max_runs), averaged.
double ref_module_time(int h, void **args, int max_runs) {
  auto &m = *g_modules[h];
  auto x = ab::recordTime(nullptr);
  m.compute(args);
  auto y = ab::recordTime(nullptr);
  double tpr = ab::convertToElapsedTime(x, y);
  if (tpr > 2) return tpr;
  unsigned long num_runs = std::max(1LU, std::min(10000LU, (unsigned long)(1.0 / tpr)));
  if (max_runs > 0 && num_runs > (unsigned long)max_runs) num_runs = max_runs;
  x = ab::recordTime(nullptr);
  for (unsigned long i = 0; i < num_runs; ++i) m.compute(args);
  y = ab::recordTime(nullptr);
  return ab::convertToElapsedTime(x, y) / num_runs;
}

// Worker threads the reference pool uses: hardware_concurrency() unless CPU_THREADS is set
// (backends/c-mcpu/include/backend.hpp:107-126).
int ref_num_threads() {
  ab::init(0);
  return (int)ab::_thread_pool->get_workers().size();
}

}  // extern "C"
