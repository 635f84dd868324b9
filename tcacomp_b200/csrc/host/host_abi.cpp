// host_abi.cpp -- the C entry points of include/tcab_host.h over ParseModule / Classify / Launch.
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../../include/tcab_host.h"
#include "tca_syntax.h"

using namespace tcab::pkg;

struct tcab_module {
  std::vector<ParsedKernel> kernels;
  mutable std::vector<std::string> described;  // one text per kernel, built on first request
};

namespace {

thread_local std::string g_error;

int fail(int status, const std::string& msg) {
  g_error = msg;
  return status;
}

const ParsedKernel* kernel_at(const tcab_module* m, uint32_t i) {
  if (m == nullptr || i >= m->kernels.size()) {
    g_error = m == nullptr ? "module is NULL" : "kernel index out of range";
    return nullptr;
  }
  return &m->kernels[i];
}

}  // namespace

extern "C" {

int tcab_module_parse(const char* text, tcab_module** out) {
  if (out == nullptr) return fail(TCAB_ERR_INVALID_ARG, "module_parse: out is NULL");
  *out = nullptr;
  if (text == nullptr) return fail(TCAB_ERR_INVALID_ARG, "module_parse: text is NULL");
  auto r = ParseModule(text);
  if (!r.ok()) {
    // constructs the reference's grammar has but this path does not evaluate say so in their message
    const bool unsupported = r.err.find("no kernel class") != std::string::npos ||
                             r.err.find("module loader") != std::string::npos;
    return fail(unsupported ? TCAB_ERR_UNSUPPORTED : TCAB_ERR_INVALID_ARG, r.err);
  }
  tcab_module* m = new tcab_module;
  m->kernels = std::move(r.value);
  *out = m;
  return TCAB_OK;
}

void tcab_module_free(tcab_module* m) { delete m; }

uint32_t tcab_module_kernel_count(const tcab_module* m) {
  return m == nullptr ? 0u : static_cast<uint32_t>(m->kernels.size());
}

const char* tcab_module_kernel_name(const tcab_module* m, uint32_t i) {
  const ParsedKernel* k = kernel_at(m, i);
  return k == nullptr ? nullptr : k->cxx_name.c_str();
}

const char* tcab_module_kernel_output(const tcab_module* m, uint32_t i) {
  const ParsedKernel* k = kernel_at(m, i);
  return k == nullptr ? nullptr : k->output.c_str();
}

const char* tcab_module_kernel_class(const tcab_module* m, uint32_t i) {
  const ParsedKernel* k = kernel_at(m, i);
  if (k == nullptr) return nullptr;
  if (k->graph.statements.empty()) {
    g_error = "kernel has no statement";
    return nullptr;
  }
  auto plan = Classify(k->graph.statements[0]);
  if (!plan.ok()) {
    g_error = plan.err;
    return nullptr;
  }
  switch (plan.value.kind) {
    case Plan::ChainReduce: return "chain_reduce";
    case Plan::ChainContract: return "chain_contract";
    case Plan::GemmBiasAct: return "gemm_bias_act";
  }
  return nullptr;
}

const char* tcab_module_kernel_describe(const tcab_module* m, uint32_t i) {
  const ParsedKernel* k = kernel_at(m, i);
  if (k == nullptr) return nullptr;
  if (k->graph.statements.empty()) {
    g_error = "kernel has no statement";
    return nullptr;
  }
  auto plan = Classify(k->graph.statements[0]);
  if (!plan.ok()) {
    g_error = plan.err;
    return nullptr;
  }
  auto join = [](const std::vector<std::string>& v) {
    std::string s;
    for (size_t j = 0; j < v.size(); ++j) s += (j ? "," : "") + v[j];
    return s;
  };
  const Plan& p = plan.value;
  std::string d;
  if (p.kind == Plan::GemmBiasAct) {
    d = "class=gemm_bias_act\nout=" + p.out + "\ninputs=" + p.a + "," + p.b + (p.bias.empty() ? "" : "," + p.bias) +
        "\na=" + p.a + "\nb=" + p.b + "\nbias=" + p.bias + "\nact=" + (p.act == TCAB_ACT_RELU ? "relu" : "none") + "\n";
  } else {
    char init[64];
    std::snprintf(init, sizeof(init), "%.9g", static_cast<double>(p.init));
    d = std::string("class=") + (p.kind == Plan::ChainReduce ? "chain_reduce" : "chain_contract") + "\nout=" + k->output +
        "\ninputs=" + join(p.inputs) + "\nmap=" + p.map_expr + "\ncombine=" + p.combine_expr + "\npost=" + p.post_expr +
        "\ninit=" + init + "\ncaptures=" + join(p.capture_names) + "\n";
    d += p.kind == Plan::ChainReduce ? "axis=" + std::to_string(p.reduce_axis) + "\n"
                                     : std::string("rhs_is_nk=") + (p.rhs_is_nk ? "1" : "0") + "\n";
  }
  {
    std::vector<std::string> names;
    for (const auto& sc : k->graph.scalars) names.push_back(sc.first);
    d += "scalars=" + join(names) + "\n";  // the kernel's scalar parameters in declaration order
  }
  if (m->described.size() < m->kernels.size()) m->described.resize(m->kernels.size());
  m->described[i] = d;
  return m->described[i].c_str();
}

int tcab_module_launch(const tcab_module* m, const char* kernel, const char* const* tensor_names,
                       const tcab_tensor* tensors, uint32_t n_tensors, const char* const* scalar_names,
                       const float* scalars, uint32_t n_scalars, void* stream) {
  if (m == nullptr || kernel == nullptr) return fail(TCAB_ERR_INVALID_ARG, "module_launch: module or kernel name is NULL");
  if ((n_tensors > 0 && (tensor_names == nullptr || tensors == nullptr)) ||
      (n_scalars > 0 && (scalar_names == nullptr || scalars == nullptr)))
    return fail(TCAB_ERR_INVALID_ARG, "module_launch: a name or value array is NULL");
  const ParsedKernel* found = nullptr;
  for (const ParsedKernel& k : m->kernels)
    if (k.cxx_name == kernel || k.name == kernel) found = &k;
  if (found == nullptr) return fail(TCAB_ERR_INVALID_ARG, std::string("module_launch: no kernel named '") + kernel + "'");
  Bindings bind;
  for (uint32_t i = 0; i < n_tensors; ++i) {
    if (tensor_names[i] == nullptr) return fail(TCAB_ERR_INVALID_ARG, "module_launch: a tensor name is NULL");
    if (!bind.tensors.emplace(tensor_names[i], tensors[i]).second)
      return fail(TCAB_ERR_INVALID_ARG, std::string("module_launch: tensor '") + tensor_names[i] + "' is bound twice");
  }
  for (uint32_t i = 0; i < n_scalars; ++i) {
    if (scalar_names[i] == nullptr) return fail(TCAB_ERR_INVALID_ARG, "module_launch: a scalar name is NULL");
    if (!bind.scalars.emplace(scalar_names[i], scalars[i]).second)
      return fail(TCAB_ERR_INVALID_ARG, std::string("module_launch: scalar '") + scalar_names[i] + "' is bound twice");
  }
  const int rc = Launch(found->graph, bind, stream);
  if (rc != TCAB_OK) g_error = LastError();
  return rc;
}

const char* tcab_host_last_error(void) { return g_error.c_str(); }

}  // extern "C"
