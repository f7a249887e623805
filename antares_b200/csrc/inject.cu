// The reference's native plugin boundary on the B200 kernel library: kernel-source text in, key
// out; key + raw tensor pointers in, launch out.
//
// Mirrors frameworks/pytorch/main_ops.cc:17-54 (`int inject(const std::string&)`,
// `void forward(int key, std::vector<Tensor>)`) and the header parse of
// graph_evaluator/execute_module.hpp:274-283: the text carries
//   // GLOBALS: name:dtype[d0, d1], ... -> name:dtype[...]
//   // BACKEND: c-b200 (device)
//   // COMPUTE_V1: - einstein_v2(input_dict={...}, extra_outputs=[...], exprss="<Antares IR>")
// (layout written by antares/antares_compiler.py:183-199, expression by
// frameworks/pytorch/custom_op.py:20-32).  Where the reference compiles the body with nvcc at the
// first call, there is nothing to compile here: the IR is matched against the operator family
// that has a hand-written sm_100a kernel (W4A16 dequantise-and-multiply, sigmoid, row softmax) and
// bound to it; any other IR is AB200_EUNSUPPORTED (no fallback).  forward() takes the tensors in
// the order of the GLOBALS line, inputs then outputs, as the reference does
// (main_ops.cc:38-42; inputs sorted by name, lang/generic.py:53-54), resolves nothing by name and
// builds no containers on the call path (contrast execute_module.hpp:322-333).
#include <mutex>
#include <regex>
#include <string>
#include <vector>

#include "common.cuh"

namespace ab200 {
namespace {

struct TensorProp {
  std::string name, dtype;
  std::vector<long> shape;
  long elems() const {
    long n = 1;
    for (long d : shape) n *= d;
    return n;
  }
};

enum { KIND_W4A16 = 1, KIND_SIGMOID = 2, KIND_SOFTMAX = 3 };

struct Module {
  int kind = 0;
  std::vector<TensorProp> ins, outs;
  // pre-resolved launch plan: argument slots and sizes
  int a_x = -1, a_q = -1, a_s = -1, a_out = -1;
  int M = 0, K = 0, N = 0, group = 0, dtype = 0;
  long n = 0;
  int rows = 0, cols = 0;
  std::string op_name;
};

std::mutex g_mu;
std::vector<Module *> g_modules;  // never shrinks: a key stays valid for the life of the process

std::vector<std::string> ssplit(const std::string &s, const std::string &sep) {
  std::vector<std::string> out;
  size_t pos = 0;
  for (;;) {
    const size_t next = s.find(sep, pos);
    if (next == std::string::npos) {
      out.push_back(s.substr(pos));
      return out;
    }
    out.push_back(s.substr(pos, next - pos));
    pos = next + sep.size();
  }
}

bool get_between(const std::string &s, const std::string &a, const std::string &b, std::string &out) {
  const size_t i = s.find(a);
  if (i == std::string::npos) return false;
  const size_t j = s.find(b, i + a.size());
  out = s.substr(i + a.size(), j == std::string::npos ? std::string::npos : j - i - a.size());
  return true;
}

// "name:dtype[d0, d1], name:dtype[d0]" with the reference's own splitting rules (execute_module.hpp:225-241)
bool parse_props(const std::string &enc, std::vector<TensorProp> &out) {
  if (enc.empty()) return true;
  for (std::string it : ssplit(enc, "], ")) {
    const size_t c = it.find(':');
    const size_t b = it.find('[');
    if (c == std::string::npos || b == std::string::npos || b < c) return false;
    TensorProp tp;
    tp.name = it.substr(0, c);
    tp.dtype = it.substr(c + 1, b - c - 1);
    std::string dims = it.substr(b + 1);
    while (!dims.empty() && (dims.back() == ']' || dims.back() == ' ' || dims.back() == '\r')) dims.pop_back();
    if (!dims.empty())
      for (const std::string &d : ssplit(dims, ", ")) {
        const long v = atol(d.c_str());
        if (v <= 0) return false;
        tp.shape.push_back(v);
      }
    out.push_back(tp);
  }
  return true;
}

std::string squash(const std::string &s) {
  std::string o;
  for (char ch : s)
    if (!isspace((unsigned char)ch)) o.push_back(ch);
  for (const char *bang : {"+=!", ">=!", "<=!"}) {
    size_t p;
    while ((p = o.find(bang)) != std::string::npos) o.erase(p + 2, 1);
  }
  return o;
}

int find_arg(const Module &m, const std::string &name, bool output) {
  const std::vector<TensorProp> &v = output ? m.outs : m.ins;
  for (size_t i = 0; i < v.size(); ++i)
    if (v[i].name == name) return (int)(i + (output ? m.ins.size() : 0));
  return -1;
}

const TensorProp &arg_prop(const Module &m, int slot) {
  return slot < (int)m.ins.size() ? m.ins[slot] : m.outs[slot - m.ins.size()];
}

int dtype_code(const std::string &d) { return d == "float16" ? AB200_F16 : d == "float32" ? AB200_F32 : -1; }

// Matches the statements against the operator family; fills the launch plan.  Patterns are the
// IR texts of samples/05_llama2_7b_int4.py:136-138, README.md:66, AntaresIR.md:226,241 with tensor
// and axis names free.
int bind(Module &m, const std::vector<std::string> &st) {
  static const std::regex w4_1(R"(^(\w+)\[(\w+),(\w+)\]=\((\w+)\[\2/8,\3\]>>\(\2%8\*4\)\)\.call\(strs\.bitwise_and,15\)\*(\w+)\[\2\]\.like\(1\)$)");
  static const std::regex w4_2(R"(^(\w+)\[(\w+),(\w+)\]=(\w+)\[\2/(\d+),\3\]\*\((\w+)\[\2,\3\]-8\)$)");
  static const std::regex w4_3(R"(^(\w+)\[(\w+)\]\+=(\w+)\[(\w+)\]\*(\w+)\[\4,\2\]\.to\(\3\.dtype\(\)\)$)");
  static const std::regex sig_readme(R"(^(\w+)\[(\w+)\]=1-1/\(1\+(\w+)\[\2\]\.call\(strs\.exp\)\)$)");
  static const std::regex sig_canon(R"(^(\w+)\[([\w,]+)\]=1\.0/\(1\.0\+\(-(\w+)\[\2\]\)\.call\(`exp`\)\)$)");
  static const std::regex sm_1(R"(^(\w+)\[(\w+)\]>=(\w+)\[\2,(\w+)\]$)");
  static const std::regex sm_2(R"(^(\w+)\[(\w+)\]\+=\((\w+)\[\2,(\w+)\]-(\w+)\[\2\]\)\.call\(`exp`\)$)");
  static const std::regex sm_3(R"(^(\w+)\[(\w+),(\w+)\]=\((\w+)\[\2,\3\]-(\w+)\[\2\]\)\.call\(`exp`\)/(\w+)\[\2\]$)");
  std::smatch a, b, c;
  if (st.size() == 3 && std::regex_match(st[0], a, w4_1) && std::regex_match(st[1], b, w4_2) && std::regex_match(st[2], c, w4_3)) {
    if (b[6] != a[1] || c[5] != b[1] || c[3] != a[5]) return fail(AB200_EUNSUPPORTED, "inject: the three W4A16 statements do not chain");
    m.a_x = find_arg(m, a[5], false);
    m.a_q = find_arg(m, a[4], false);
    m.a_s = find_arg(m, b[4], false);
    m.a_out = find_arg(m, c[1], true);
    if (m.a_x < 0 || m.a_q < 0 || m.a_s < 0 || m.a_out < 0) return fail(AB200_EINVAL, "inject: a W4A16 tensor is missing from the GLOBALS line");
    const TensorProp &x = arg_prop(m, m.a_x), &q = arg_prop(m, m.a_q), &s = arg_prop(m, m.a_s), &o = arg_prop(m, m.a_out);
    if (q.dtype != "int32" || q.shape.size() != 2 || s.shape.size() != 2 || x.shape.empty())
      return fail(AB200_EUNSUPPORTED, "inject: W4A16 wants qweight int32 [K/8, N], scales [K/group, N]");
    m.dtype = dtype_code(x.dtype);
    if (m.dtype < 0 || s.dtype != x.dtype || o.dtype != x.dtype)
      return fail(AB200_EUNSUPPORTED, "inject: W4A16 activations, scales and result must all be float16 or all float32");
    m.K = (int)q.shape[0] * 8;
    m.N = (int)q.shape[1];
    m.group = atoi(b[5].str().c_str());
    if (x.shape.back() != m.K || x.elems() % m.K) return fail(AB200_EINVAL, "inject: activations have %ld values per row, the weights %d rows", x.shape.back(), m.K);
    m.M = (int)(x.elems() / m.K);
    if (m.group <= 0 || m.K % m.group || s.shape[0] != m.K / m.group || s.shape[1] != m.N || o.elems() != (long)m.M * m.N)
      return fail(AB200_EINVAL, "inject: W4A16 shapes disagree (K=%d N=%d group=%d M=%d)", m.K, m.N, m.group, m.M);
    m.kind = KIND_W4A16;
    m.op_name = c[1];
    return AB200_OK;
  }
  if (st.size() == 3 && std::regex_match(st[0], a, sm_1) && std::regex_match(st[1], b, sm_2) && std::regex_match(st[2], c, sm_3)) {
    if (a[3] != b[3] || a[3] != c[4] || b[5] != a[1] || c[5] != a[1] || c[6] != b[1]) return fail(AB200_EUNSUPPORTED, "inject: the three softmax statements do not chain");
    m.a_x = find_arg(m, a[3], false);
    m.a_out = find_arg(m, c[1], true);
    if (m.a_x < 0 || m.a_out < 0) return fail(AB200_EINVAL, "inject: a softmax tensor is missing from the GLOBALS line");
    const TensorProp &x = arg_prop(m, m.a_x), &o = arg_prop(m, m.a_out);
    m.dtype = dtype_code(x.dtype);
    if (m.dtype < 0 || o.dtype != x.dtype || x.shape.size() != 2 || o.shape != x.shape) return fail(AB200_EUNSUPPORTED, "inject: softmax wants one float16/float32 [rows, cols] tensor in and out");
    m.rows = (int)x.shape[0];
    m.cols = (int)x.shape[1];
    m.kind = KIND_SOFTMAX;
    m.op_name = c[1];
    return AB200_OK;
  }
  if (st.size() == 1 && (std::regex_match(st[0], a, sig_readme) || std::regex_match(st[0], a, sig_canon))) {
    m.a_x = find_arg(m, a[3], false);
    m.a_out = find_arg(m, a[1], true);
    if (m.a_x < 0 || m.a_out < 0) return fail(AB200_EINVAL, "inject: a sigmoid tensor is missing from the GLOBALS line");
    const TensorProp &x = arg_prop(m, m.a_x), &o = arg_prop(m, m.a_out);
    m.dtype = dtype_code(x.dtype);
    if (m.dtype < 0 || o.dtype != x.dtype || o.elems() != x.elems()) return fail(AB200_EUNSUPPORTED, "inject: sigmoid wants float16/float32 tensors of one size");
    m.n = x.elems();
    m.kind = KIND_SIGMOID;
    m.op_name = a[1];
    return AB200_OK;
  }
  return fail(AB200_EUNSUPPORTED,
              "inject: this IR is outside the operator family with hand-written kernels (W4A16 dequantise-and-multiply, sigmoid, row softmax); "
              "there is no code generator and no fallback");
}

int inject_impl(const std::string &src, int *key_out) {
  std::string globals, backend, compute;
  if (!get_between(src, "// GLOBALS: ", "\n", globals)) return fail(AB200_EINVAL, "inject: no `// GLOBALS:` line");
  if (!get_between(src, "// BACKEND: ", " (", backend)) return fail(AB200_EINVAL, "inject: no `// BACKEND:` line");
  if (backend != "c-b200") return fail(AB200_EUNSUPPORTED, "inject: backend `%s` (this library serves `c-b200`)", backend.c_str());
  if (!get_between(src, "// COMPUTE_V1: ", "\n", compute)) return fail(AB200_EINVAL, "inject: no `// COMPUTE_V1:` line");
  const std::vector<std::string> io = ssplit(globals, " -> ");
  if (io.size() != 2) return fail(AB200_EINVAL, "inject: the GLOBALS line needs `inputs -> outputs`");
  Module *m = new Module();
  if (!parse_props(io[0], m->ins) || !parse_props(io[1], m->outs) || m->outs.empty()) {
    delete m;
    return fail(AB200_EINVAL, "inject: cannot parse the GLOBALS line `%s`", globals.c_str());
  }
  // the IR text: exprss="..." (custom_op.py:31) or the first string argument of einstein_v2(
  std::string ir;
  size_t p = compute.find("exprss=\"");
  if (p != std::string::npos) p += 8;
  else {
    p = compute.find("einstein_v2(");
    if (p != std::string::npos) p = compute.find('"', p);
    if (p != std::string::npos) p += 1;
  }
  if (p == std::string::npos) {
    delete m;
    return fail(AB200_EINVAL, "inject: no einstein_v2(...) expression in the COMPUTE_V1 line");
  }
  const size_t e = compute.find('"', p);
  ir = compute.substr(p, e == std::string::npos ? std::string::npos : e - p);
  std::vector<std::string> st;
  for (const std::string &piece : ssplit(ir, ";")) {
    const std::string s = squash(piece);
    if (!s.empty()) st.push_back(s);
  }
  if (st.empty()) {
    delete m;
    return fail(AB200_EINVAL, "inject: empty IR");
  }
  if (int rc = bind(*m, st)) {
    delete m;
    return rc;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  g_modules.push_back(m);
  *key_out = (int)g_modules.size() - 1;
  return AB200_OK;
}

inline const Module *lookup(int key) {
  // keys index an append-only table of heap objects: a reader needs the lock only for the table itself
  std::lock_guard<std::mutex> lk(g_mu);
  return (key >= 0 && key < (int)g_modules.size()) ? g_modules[key] : nullptr;
}

inline int forward_impl(const Module *m, void *const *args, int n_args, void *stream) {
  if (n_args != (int)(m->ins.size() + m->outs.size()))
    return fail(AB200_EINVAL, "forward: %d arguments, the module declares %zu inputs + %zu outputs", n_args, m->ins.size(), m->outs.size());
  switch (m->kind) {
    case KIND_W4A16:
      if (m->M <= 16)
        return ab200_w4a16_gemv(args[m->a_x], (const int32_t *)args[m->a_q], args[m->a_s], args[m->a_out], m->M, m->K, m->N, m->group, m->dtype, stream);
      return ab200_w4a16_gemm(args[m->a_x], (const int32_t *)args[m->a_q], args[m->a_s], args[m->a_out], m->M, m->K, m->N, m->group, m->dtype, stream);
    case KIND_SIGMOID:
      return ab200_sigmoid(args[m->a_x], args[m->a_out], (size_t)m->n, m->dtype, stream);
    case KIND_SOFTMAX:
      return ab200_softmax(args[m->a_x], args[m->a_out], m->rows, m->cols, m->dtype, stream);
  }
  return fail(AB200_EINVAL, "forward: module has no kernel bound");
}

}  // namespace
}  // namespace ab200

using namespace ab200;

extern "C" int ab200_inject(const char *source, int *key_out) {
  clear_error();
  AB200_REQUIRE(source && key_out, "inject: null argument");
  try {
    return inject_impl(std::string(source), key_out);
  } catch (const std::exception &e) {
    return fail(AB200_EINVAL, "inject: %s", e.what());
  }
}

extern "C" int ab200_forward(int key, void *const *args_host, int n_args, void *stream) {
  const Module *m = lookup(key);
  if (!m) {
    clear_error();
    return fail(AB200_EINVAL, "forward: unknown key %d", key);
  }
  if (!args_host) {
    clear_error();
    return fail(AB200_EINVAL, "forward: null argument array");
  }
  return forward_impl(m, args_host, n_args, stream);
}

extern "C" int ab200_module_info(int key, int *n_inputs_host, int *n_outputs_host, char *op_name_host, int op_name_cap) {
  clear_error();
  const Module *m = lookup(key);
  AB200_REQUIRE(m != nullptr, "module_info: unknown key %d", key);
  if (n_inputs_host) *n_inputs_host = (int)m->ins.size();
  if (n_outputs_host) *n_outputs_host = (int)m->outs.size();
  if (op_name_host && op_name_cap > 0) snprintf(op_name_host, op_name_cap, "%s", m->op_name.c_str());
  return AB200_OK;
}

extern "C" int ab200_module_tensor(int key, int slot, char *name_host, int name_cap, char *dtype_host, int dtype_cap, long *shape8_host, int *rank_host) {
  clear_error();
  const Module *m = lookup(key);
  AB200_REQUIRE(m != nullptr, "module_tensor: unknown key %d", key);
  AB200_REQUIRE(slot >= 0 && slot < (int)(m->ins.size() + m->outs.size()), "module_tensor: slot %d out of range", slot);
  const TensorProp &t = arg_prop(*m, slot);
  AB200_REQUIRE(t.shape.size() <= 8, "module_tensor: rank above 8");
  if (name_host && name_cap > 0) snprintf(name_host, name_cap, "%s", t.name.c_str());
  if (dtype_host && dtype_cap > 0) snprintf(dtype_host, dtype_cap, "%s", t.dtype.c_str());
  if (rank_host) *rank_host = (int)t.shape.size();
  if (shape8_host)
    for (size_t i = 0; i < t.shape.size(); ++i) shape8_host[i] = t.shape[i];
  return AB200_OK;
}

// Host cost of the call path itself: `iters` forward() calls back to back on one stream, wall
// time per call in nanoseconds (the launches queue up; nothing is synchronised inside the loop).
extern "C" int ab200_forward_host_ns(int key, void *const *args_host, int n_args, void *stream, int iters, double *ns_per_call_host) {
  clear_error();
  const Module *m = lookup(key);
  AB200_REQUIRE(m != nullptr && args_host && ns_per_call_host && iters > 0, "forward_host_ns: bad argument");
  timespec t0, t1;
  clock_gettime(CLOCK_MONOTONIC, &t0);
  for (int i = 0; i < iters; ++i)
    if (int rc = ab200_forward(key, args_host, n_args, stream)) return rc;
  clock_gettime(CLOCK_MONOTONIC, &t1);
  *ns_per_call_host = ((t1.tv_sec - t0.tv_sec) * 1e9 + (t1.tv_nsec - t0.tv_nsec)) / iters;
  return AB200_OK;
}
