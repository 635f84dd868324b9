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
  mutable std::vector<std::string> classes;
  mutable std::vector<std::string> signatures;
};

namespace {

thread_local std::string g_error;

int fail(int status, const std::string& msg) {
  g_error = msg;
  return status;
}

const char* class_name(Plan::Kind k) {
  switch (k) {
    case Plan::ChainReduce: return "chain_reduce";
    case Plan::ChainContract: return "chain_contract";
    case Plan::GemmBiasAct: return "gemm_bias_act";
    case Plan::Map: return "map";
    case Plan::SoftmaxRows: return "softmax_rows";
    case Plan::LayernormRows: return "layernorm_rows";
  }
  return "";
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
    const bool unsupported = r.err.find("no kernel class") != std::string::npos;
    return fail(unsupported ? TCAB_ERR_UNSUPPORTED : TCAB_ERR_INVALID_ARG, r.err);
  }
  tcab_module* m = new tcab_module;
  m->kernels = std::move(r.value);
  *out = m;
  return TCAB_OK;
}

int tcab_module_parse_files(const char* const* paths, const char* const* texts, uint32_t n_files, const char* root,
                            tcab_module** out) {
  if (out == nullptr) return fail(TCAB_ERR_INVALID_ARG, "module_parse_files: out is NULL");
  *out = nullptr;
  if (paths == nullptr || texts == nullptr || root == nullptr || n_files == 0)
    return fail(TCAB_ERR_INVALID_ARG, "module_parse_files: paths, texts and root are required");
  std::vector<SourceFile> files;
  for (uint32_t i = 0; i < n_files; ++i) {
    if (paths[i] == nullptr || texts[i] == nullptr) return fail(TCAB_ERR_INVALID_ARG, "module_parse_files: a path or text is NULL");
    files.push_back(SourceFile{paths[i], texts[i]});
  }
  auto r = ParseModuleFiles(files, root);
  if (!r.ok()) return fail(r.err.find("no kernel class") != std::string::npos ? TCAB_ERR_UNSUPPORTED : TCAB_ERR_INVALID_ARG, r.err);
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
  auto plans = PlanGraph(k->graph);
  if (!plans.ok()) {
    g_error = plans.err;
    return nullptr;
  }
  std::string cls;
  for (const Plan& p : plans.value) cls += (cls.empty() ? "" : "+") + std::string(class_name(p.kind));
  if (m->classes.size() < m->kernels.size()) m->classes.resize(m->kernels.size());
  m->classes[i] = cls;
  return m->classes[i].c_str();
}

const char* tcab_module_kernel_describe(const tcab_module* m, uint32_t i) {
  const ParsedKernel* k = kernel_at(m, i);
  if (k == nullptr) return nullptr;
  if (k->graph.statements.empty()) {
    g_error = "kernel has no statement";
    return nullptr;
  }
  auto plans = PlanGraph(k->graph);
  if (!plans.ok()) {
    g_error = plans.err;
    return nullptr;
  }
  auto join = [](const std::vector<std::string>& v) {
    std::string s;
    for (size_t j = 0; j < v.size(); ++j) s += (j ? "," : "") + v[j];
    return s;
  };
  auto one = [&](const Plan& p, const std::string& out_name, const std::string& pre) {
    std::string d;
    if (p.kind == Plan::GemmBiasAct) {
      d = pre + "class=gemm_bias_act\n" + pre + "out=" + p.out + "\n" + pre + "inputs=" + p.a + "," + p.b +
          (p.bias.empty() ? "" : "," + p.bias) + "\n" + pre + "a=" + p.a + "\n" + pre + "b=" + p.b + "\n" + pre + "bias=" + p.bias +
          "\n" + pre + "act=" + (p.act == TCAB_ACT_RELU ? "relu" : "none") + "\n";
    } else if (p.kind == Plan::SoftmaxRows || p.kind == Plan::LayernormRows) {
      d = pre + "class=" + class_name(p.kind) + "\n" + pre + "out=" + out_name + "\n" + pre + "inputs=" + join(p.inputs) + "\n" +
          pre + "fused_locals=" + join(p.fused_locals) + "\n";
      if (p.kind == Plan::LayernormRows) d += pre + "eps=" + p.eps_scalar + "\n" + pre + "inv_n=" + p.capture_names[0] + "\n";
    } else {
      char init[64];
      std::snprintf(init, sizeof(init), "%.9g", static_cast<double>(p.init));
      d = pre + "class=" + class_name(p.kind) + "\n" + pre + "out=" + out_name + "\n" + pre + "inputs=" + join(p.inputs) + "\n" +
          pre + "map=" + p.map_expr + "\n";
      if (p.kind != Plan::Map)
        d += pre + "combine=" + p.combine_expr + "\n" + pre + "post=" + p.post_expr + "\n" + pre + "init=" + init + "\n";
      d += pre + "captures=" + join(p.capture_names) + "\n";
      if (p.kind == Plan::ChainReduce) d += pre + "axis=" + std::to_string(p.reduce_axis) + "\n";
      if (p.kind == Plan::ChainContract) d += pre + std::string("rhs_is_nk=") + (p.rhs_is_nk ? "1" : "0") + "\n";
      bool subset = false;
      for (int h : p.indexing) subset = subset || h != 0;
      if (subset) {   // how each operand is indexed: 0 every axis, 1 one value per row, 2 one row shared by all rows
        std::vector<std::string> hs;
        for (int h : p.indexing) hs.push_back(std::to_string(h));
        d += pre + "indexing=" + join(hs) + "\n";
      }
    }
    return d;
  };
  std::string d;
  if (plans.value.size() == 1) {
    d = one(plans.value[0], k->output, "");
  } else {
    std::string cls;
    for (const Plan& p : plans.value) cls += (cls.empty() ? "" : "+") + std::string(class_name(p.kind));
    d = "class=" + cls + "\nout=" + k->output + "\nlaunches=" + std::to_string(plans.value.size()) + "\n";
    for (size_t j = 0; j < plans.value.size(); ++j) d += one(plans.value[j], plans.value[j].out, "launch" + std::to_string(j) + ".");
  }
  {
    // the intermediates between statements that still need device memory from the caller (a local of a statement
    // group that was replaced by one launch needs none), each with its element type and dims
    std::vector<std::string> fused, need;
    for (const Plan& p : plans.value) fused.insert(fused.end(), p.fused_locals.begin(), p.fused_locals.end());
    std::string shapes;
    for (const Tensor& t : k->graph.tensors) {
      if (!t.local) continue;
      bool gone = false;
      for (const std::string& f : fused) gone = gone || f == t.name;
      if (gone) continue;
      need.push_back(t.name);
      std::vector<std::string> dn;
      for (const Dim& dm : t.dims) dn.push_back(dm.extent > 0 ? std::to_string(dm.extent) : dm.name);
      shapes += "local." + t.name + "=" + ElemName(t.elem) + "[" + join(dn) + "]\n";
    }
    if (plans.value.size() > 1 || !need.empty()) d += "locals=" + join(need) + "\n" + shapes;
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

const char* tcab_module_kernel_signature(const tcab_module* m, uint32_t i) {
  const ParsedKernel* k = kernel_at(m, i);
  if (k == nullptr) return nullptr;
  std::string d;
  for (const Tensor& t : k->graph.tensors) {
    d += t.name + "=" + ElemName(t.elem) + "[";
    for (size_t j = 0; j < t.dims.size(); ++j)
      d += (j ? "," : "") + (t.dims[j].extent > 0 ? std::to_string(t.dims[j].extent) : t.dims[j].name);
    d += t.local ? "] local\n" : "]\n";
  }
  for (const auto& sc : k->graph.scalars) d += sc.first + "=" + ElemName(sc.second) + "\n";
  if (m->signatures.size() < m->kernels.size()) m->signatures.resize(m->kernels.size());
  m->signatures[i] = d;
  return m->signatures[i].c_str();
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
