// chain_jit.cu -- run-time compilation of the chain kernels for lambdas that have no
// ahead-of-time instance.
//
// The reference compiles every kernel from its lambdas (internal/cg/cxx/emit.go:85-190 prints the
// translation unit, the user runs nvcc). Here the kernels are fixed text (chain_kernels.cuh, embedded
// in the library at build time) and only the two functor structs are printed from the caller's
// canonical lambda text, which expr.cpp has validated token by token: nothing but + - * /, unary
// minus, p#/c# and the reference's fp32 builtins can appear in it. NVRTC (libnvrtc, opened with
// dlopen on first need) compiles that for sm_100a; the cubin is loaded once per process with
// cudaLibraryLoadData and cached by lambda text. Compilation happens on the first call with a new
// lambda (a few hundred milliseconds); later calls only look the kernels up.
#include <dlfcn.h>
#include <nvrtc.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "chain_kernels.cuh"
#include "common.cuh"

namespace tcab {
namespace {

const char kKernelText[] =
#include "chain_kernels_text.inc"
    ;

struct Nvrtc {
  void* handle = nullptr;
  decltype(&nvrtcCreateProgram) create = nullptr;
  decltype(&nvrtcDestroyProgram) destroy = nullptr;
  decltype(&nvrtcCompileProgram) compile = nullptr;
  decltype(&nvrtcAddNameExpression) add_name = nullptr;
  decltype(&nvrtcGetLoweredName) lowered = nullptr;
  decltype(&nvrtcGetCUBINSize) cubin_size = nullptr;
  decltype(&nvrtcGetCUBIN) cubin = nullptr;
  decltype(&nvrtcGetProgramLogSize) log_size = nullptr;
  decltype(&nvrtcGetProgramLog) log = nullptr;
  bool ok = false;
};

const Nvrtc& nvrtc() {
  static Nvrtc n;
  static std::once_flag once;
  std::call_once(once, [] {
    for (const char* name : {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12"}) {
      n.handle = dlopen(name, RTLD_NOW | RTLD_LOCAL);
      if (n.handle) break;
    }
    if (!n.handle) return;
#define TCAB_SYM(field, sym) n.field = reinterpret_cast<decltype(n.field)>(dlsym(n.handle, #sym))
    TCAB_SYM(create, nvrtcCreateProgram);
    TCAB_SYM(destroy, nvrtcDestroyProgram);
    TCAB_SYM(compile, nvrtcCompileProgram);
    TCAB_SYM(add_name, nvrtcAddNameExpression);
    TCAB_SYM(lowered, nvrtcGetLoweredName);
    TCAB_SYM(cubin_size, nvrtcGetCUBINSize);
    TCAB_SYM(cubin, nvrtcGetCUBIN);
    TCAB_SYM(log_size, nvrtcGetProgramLogSize);
    TCAB_SYM(log, nvrtcGetProgramLog);
#undef TCAB_SYM
    n.ok = n.create && n.destroy && n.compile && n.add_name && n.lowered && n.cubin_size && n.cubin && n.log_size &&
           n.log;
  });
  return n;
}

// The kernels one chain needs, in the order of JitChain::k.
enum Slot {
  kInner1V4, kInner4V4, kInner32V4, kInner256V4, kInner1V1, kInner4V1, kInner32V1, kInner256V1,
  kSplitV4, kSplitV1, kFinish, kOuterV4, kOuterV1, kContractKN, kContractNK, kContractKN8, kContractNK8, kMap8, kMap1,
  kInner32V4Big, kBatch32V4, kBatch256V4, kBatch32V1, kBatch256V1, kOuterFlat, kOuterFlat1, kInner4V8, kInner32V8, kInner256V8, kSplitV8, kInnerRag4, kInnerRag32, kInnerRag256, kInnerRows32e, kInnerFlat, kInnerFlat2, kInnerRows32, kSlots
};

struct JitChain {
  cudaLibrary_t lib = nullptr;
  cudaKernel_t k[kSlots] = {};
  int n_in = 0;
  char kind = 'R';
  bool broadcast = false;  // an operand is not indexed by every axis: innermost-axis kernels only
  bool cells = false;      // an operand lacks the reduced middle axis: middle-axis kernels only
  bool all_bf16 = false;   // every operand is bf16: kernels on vectors of eight exist
};

std::mutex g_mu;
std::map<std::string, JitChain*> g_cache;   // key: R or C | n_in | combine | map text | post text
std::map<std::string, std::string> g_failed;  // key -> compiler message (do not recompile a failing lambda)

// A lambda as a functor over the kernels' 32-bit operand registers (see chain_kernels.cuh): the prologue gives
// every operand its declared type back, the body is the canonical text, and the value returns as an f32
// register again (an integer as its bit pattern, a bf16 widened exactly).
std::string functor(const char* name, const std::string& expr, int n_in, const int* in_types, int result_type) {
  std::string s = "struct ";
  s += name;
  s += " {\n  static __device__ __forceinline__ float apply(const float* p, const float* c) {\n";
  for (int i = 0; i < n_in; ++i) {
    const std::string pi = "p" + std::to_string(i), src = "p[" + std::to_string(i) + "]";
    switch (in_types ? in_types[i] : TCAB_F32) {
      case TCAB_BF16: s += "    const __nv_bfloat16 " + pi + " = __nv_bfloat16::widened(" + src + ");\n"; break;
      case TCAB_I32: s += "    const int32_t " + pi + " = __float_as_int(" + src + ");\n"; break;
      case TCAB_U32: s += "    const uint32_t " + pi + " = __float_as_uint(" + src + ");\n"; break;
      default: s += "    const float " + pi + " = " + src + ";\n"; break;
    }
    s += "    (void)" + pi + ";\n";
  }
  for (int i = 0; i < 8; ++i) s += "    const float c" + std::to_string(i) + " = c[" + std::to_string(i) + "];\n";
  s += "    (void)c0; (void)c1; (void)c2; (void)c3; (void)c4; (void)c5; (void)c6; (void)c7;\n";
  switch (result_type) {
    case TCAB_BF16: s += "    return static_cast<float>(" + expr + ");\n"; break;
    case TCAB_I32: s += "    return __int_as_float(" + expr + ");\n"; break;
    case TCAB_U32: s += "    return __uint_as_float(" + expr + ");\n"; break;
    default: s += "    return " + expr + ";\n"; break;
  }
  s += "  }\n};\n";
  return s;
}

// One program per chain and use: the reduction kernels (13 instances), the contraction kernels (4) or the
// map-only kernels (2), never more than one group -- a chain is launched through one entry point, and the
// unrolled contraction tiles are the slowest instances to compile.
int compile(const std::string& key, const JitSpec& sp, JitChain** out, bool load = true) {
  const std::string &map_text = sp.map_text, &post_text = sp.post_text;
  const Nvrtc& nv = nvrtc();
  if (!nv.ok)
    return fail(TCAB_ERR_UNSUPPORTED,
                "chain: no kernel in this build for map '%s' post '%s', and libnvrtc is not available to "
                "compile one", map_text.c_str(), post_text.c_str());
  std::string src = kKernelText;
  // the element types' C++ spellings as the reference emits them (internal/cg/cxx/naming.go:21-46)
  src += "\nnamespace tcabj {\ntypedef tcabk::bf16 __nv_bfloat16;\ntypedef int int32_t;\ntypedef unsigned int uint32_t;\n";
  src += functor("Map", map_text, sp.n_in, sp.in_types, sp.kind == 'M' ? sp.out_type : TCAB_F32);
  src += post_text.empty() ? "typedef tcabk::PostNone Post;\n" : functor("Post", post_text, 1, nullptr, TCAB_F32);
  src += "}\n";
  const std::string n = std::to_string(sp.n_in), c = std::to_string(sp.combine), bf = std::to_string(sp.bf_mask());
  const std::string bc = ", " + std::to_string(sp.rb_mask) + ", " + std::to_string(sp.cb_mask);  // broadcast masks
  std::vector<std::string> names(kSlots);
  if (sp.kind == 'R') {
    const int tprs[4] = {1, 4, 32, 256};
    for (int v = 0; v < 2; ++v)
      for (int t = 0; t < 4; ++t)
        names[(v == 0 ? kInner1V4 : kInner1V1) + t] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", " +
                                                      std::to_string(tprs[t]) + ", " + (v == 0 ? "4" : "1") + ", " + bf + ", " +
                                                      std::to_string(tprs[t] > 128 ? tprs[t] : 128) + bc + ">";
    names[kInner32V4Big] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 32, 4, " + bf + ", 1024" + bc + ">";
    if (sp.cell_mask != 0) {  // operands without the reduced middle axis: the middle-axis kernels only
      names.assign(kSlots, std::string());
      const std::string cm = ", " + std::to_string(sp.cell_mask);
      names[kFinish] = "tcabk::chain_split_finish<tcabj::Post, " + c + ">";
      names[kOuterV4] = "tcabk::chain_outer<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 4, 8, 4, " + bf + cm + ">";
      names[kOuterV1] = "tcabk::chain_outer<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 1, 8, 8, " + bf + cm + ">";
      names[kOuterFlat] = "tcabk::chain_outer_flat<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 4, " + bf + cm + ">";
      names[kOuterFlat1] = "tcabk::chain_outer_flat<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 16, " + bf + cm + ", 1>";
    } else if ((sp.rb_mask | sp.cb_mask) != 0) {  // broadcast operands: the innermost-axis kernels only
      names.assign(kSlots, std::string());
      for (int v = 0; v < 2; ++v)
        for (int t = 0; t < 4; ++t)
          names[(v == 0 ? kInner1V4 : kInner1V1) + t] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", " +
                                                        std::to_string(tprs[t]) + ", " + (v == 0 ? "4" : "1") + ", " + bf + ", " +
                                                        std::to_string(tprs[t] > 128 ? tprs[t] : 128) + bc + ">";
      names[kInner32V4Big] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 32, 4, " + bf + ", 1024" + bc + ">";
      if (sp.bf_mask() == (1 << sp.n_in) - 1) {  // every operand bf16: vectors of eight, as without broadcast operands
        names[kInner4V8] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 4, 8, " + bf + ", 128" + bc + ">";
        names[kInner32V8] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 32, 8, " + bf + ", 128" + bc + ">";
        names[kInner256V8] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 256, 8, " + bf + ", 256" + bc + ">";
      }
    } else {
    names[kSplitV4] = "tcabk::chain_inner_split<tcabj::Map, " + c + ", " + n + ", 4, " + bf + ">";
    names[kSplitV1] = "tcabk::chain_inner_split<tcabj::Map, " + c + ", " + n + ", 1, " + bf + ">";
    names[kFinish] = "tcabk::chain_split_finish<tcabj::Post, " + c + ">";
    names[kOuterV4] = "tcabk::chain_outer<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 4, 8, 4, " + bf + ">";
    names[kOuterV1] = "tcabk::chain_outer<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 1, 8, 8, " + bf + ">";
    names[kOuterFlat] = "tcabk::chain_outer_flat<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 4, " + bf + ">";
    names[kOuterFlat1] = "tcabk::chain_outer_flat<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 16, " + bf + ", 0, 1>";
    names[kInnerFlat] = "tcabk::chain_inner_flat<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 4, " + bf + ">";
    names[kInnerFlat2] = "tcabk::chain_inner_flat<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 4, " + bf + ", 2>";
    names[kInnerRows32] = "tcabk::chain_inner_rows32<tcabj::Map, tcabj::Post, " + c + ", " + n + ", " + bf + ">";
    if (sp.n_in > 0 && sp.bf_mask() == (1 << sp.n_in) - 1) {  // every operand bf16: 16-byte loads are vectors of eight
      names[kInner4V8] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 4, 8, " + bf + ", 128>";
      names[kInner32V8] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 32, 8, " + bf + ", 128>";
      names[kInner256V8] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 256, 8, " + bf + ", 256>";
      names[kSplitV8] = "tcabk::chain_inner_split<tcabj::Map, " + c + ", " + n + ", 8, " + bf + ">";
    }
    names[kInnerRows32e] = "tcabk::chain_inner_rows32e<tcabj::Map, tcabj::Post, " + c + ", " + n + ", " + bf + ">";
    names[kInnerRag4] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 4, 4, " + bf + ", 128, 0, 0, 1>";
    names[kInnerRag32] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 32, 4, " + bf + ", 128, 0, 0, 1>";
    names[kInnerRag256] = "tcabk::chain_inner<tcabj::Map, tcabj::Post, " + c + ", " + n + ", 256, 4, " + bf + ", 256, 0, 0, 1>";
    }
  } else if (sp.kind == 'B') {
    const char* shapes[4] = {"32, 4", "256, 4", "32, 1", "256, 1"};
    for (int i = 0; i < 4; ++i)
      names[kBatch32V4 + i] = "tcabk::chain_inner_batched<tcabj::Map, tcabj::Post, " + c + ", " + n + ", " + shapes[i] + ", " + bf + ">";
  } else if (sp.kind == 'C') {
    names[kContractKN] = "tcabk::chain_contract<tcabj::Map, tcabj::Post, " + c + ", 0, 4, " + bf + ">";
    names[kContractNK] = "tcabk::chain_contract<tcabj::Map, tcabj::Post, " + c + ", 1, 4, " + bf + ">";
    names[kContractKN8] = "tcabk::chain_contract<tcabj::Map, tcabj::Post, " + c + ", 0, 8, " + bf + ">";
    names[kContractNK8] = "tcabk::chain_contract<tcabj::Map, tcabj::Post, " + c + ", 1, 8, " + bf + ">";
  } else {
    const std::string ob = sp.out_type == TCAB_BF16 ? "true" : "false";
    names[kMap8] = "tcabk::chain_map<tcabj::Map, " + n + ", " + bf + ", " + ob + ", 8" + bc + ">";
    names[kMap1] = "tcabk::chain_map<tcabj::Map, " + n + ", " + bf + ", " + ob + ", 1" + bc + ">";
  }

  nvrtcProgram prog = nullptr;
  if (nv.create(&prog, src.c_str(), "tcab_chain_jit.cu", 0, nullptr, nullptr) != NVRTC_SUCCESS)
    return fail(TCAB_ERR_CUDA, "chain_reduce: nvrtcCreateProgram failed");
  for (const std::string& e : names)
    if (!e.empty()) nv.add_name(prog, e.c_str());
  const char* opts[] = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo"};
  const nvrtcResult res = nv.compile(prog, 3, opts);
  if (res != NVRTC_SUCCESS) {
    size_t ls = 0;
    nv.log_size(prog, &ls);
    std::string log(ls, '\0');
    if (ls) nv.log(prog, &log[0]);
    nv.destroy(&prog);
    if (load) g_failed[key] = log.substr(0, 300);
    return fail(TCAB_ERR_UNSUPPORTED, "chain_reduce: run-time compilation of map '%s' post '%s' failed: %s",
                map_text.c_str(), post_text.c_str(), log.substr(0, 300).c_str());
  }
  if (!load) {  // a compile check on a host without a device: the image is not loaded
    nv.destroy(&prog);
    return TCAB_OK;
  }
  size_t cs = 0;
  nv.cubin_size(prog, &cs);
  std::vector<char> cubin(cs);
  nv.cubin(prog, cubin.data());
  auto* jc = new JitChain();
  jc->n_in = sp.n_in;
  jc->kind = sp.kind;
  jc->broadcast = (sp.rb_mask | sp.cb_mask) != 0;
  jc->cells = sp.cell_mask != 0;
  jc->all_bf16 = sp.n_in > 0 && sp.bf_mask() == (1 << sp.n_in) - 1;
  cudaError_t e = cudaLibraryLoadData(&jc->lib, cubin.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
  for (int i = 0; e == cudaSuccess && i < static_cast<int>(names.size()); ++i) {
    if (names[i].empty()) continue;
    const char* low = nullptr;
    if (nv.lowered(prog, names[i].c_str(), &low) != NVRTC_SUCCESS || low == nullptr) {
      e = cudaErrorSymbolNotFound;
      break;
    }
    e = cudaLibraryGetKernel(&jc->k[i], jc->lib, low);
  }
  nv.destroy(&prog);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (jc->lib) cudaLibraryUnload(jc->lib);
    delete jc;
    return fail(TCAB_ERR_CUDA, "chain_reduce: loading the compiled kernels failed: %s", cudaGetErrorString(e));
  }
  *out = jc;
  return TCAB_OK;
}

int launch(cudaKernel_t k, uint64_t grid, unsigned block, void** args, cudaStream_t s, const char* what, size_t smem = 0) {
  if (grid > 0x7fffffffull) grid = 0x7fffffffull;
  const cudaError_t e = cudaLaunchKernel(reinterpret_cast<const void*>(k), dim3(static_cast<unsigned>(grid)),
                                         dim3(block), args, smem, s);
  count_launch();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
  }
  return TCAB_OK;
}

}  // namespace

bool jit_available() { return nvrtc().ok; }

int jit_prepare(const JitSpec& sp, void** handle, bool compile_if_missing) {
  const std::string& map_text = sp.map_text;
  std::string key(1, sp.kind);
  key += "|" + std::to_string(sp.n_in) + "|" + std::to_string(sp.combine) + "|";
  for (int i = 0; i < sp.n_in; ++i) key += std::to_string(sp.in_types[i]);
  key += ">" + std::to_string(sp.kind == 'M' ? sp.out_type : TCAB_F32) + "|" + std::to_string(sp.rb_mask) + "," +
         std::to_string(sp.cb_mask) + "," + std::to_string(sp.cell_mask) + "|" + sp.map_text + "|" + sp.post_text;
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_cache.find(key);
  if (it != g_cache.end()) {
    *handle = it->second;
    return TCAB_OK;
  }
  auto f = g_failed.find(key);
  if (f != g_failed.end())
    return fail(TCAB_ERR_UNSUPPORTED, "chain_reduce: run-time compilation of map '%s' failed earlier: %s",
                map_text.c_str(), f->second.c_str());
  if (!compile_if_missing) return fail(TCAB_ERR_UNSUPPORTED, "chain: lambda '%s' is not compiled yet", map_text.c_str());
  JitChain* jc = nullptr;
  const int rc = compile(key, sp, &jc);
  if (rc != TCAB_OK) return rc;
  g_cache[key] = jc;
  *handle = jc;
  return TCAB_OK;
}

int jit_compile_check(const JitSpec& sp) {
  std::lock_guard<std::mutex> lk(g_mu);
  JitChain* none = nullptr;
  return compile("check", sp, &none, false);
}

// Mirrors the ahead-of-time dispatch of chain_reduce.cu (launch_chain / launch_split / launch_outer).
// The second launch of a split reduction (several threads per output when it has many partials: finish_lanes).
static int launch_jit_finish(JitChain* jc, float* scratch, float* out, uint32_t rows, uint32_t splits, float init,
                             tcabk::Caps caps, cudaStream_t s) {
  uint32_t lanes = finish_lanes(splits);
  void* a2[] = {&scratch, &out, &rows, &splits, &init, &caps, &lanes};
  return launch(jc->k[kFinish], (static_cast<uint64_t>(rows) * lanes + 127) / 128, 128, a2, s, "chain_split_finish");
}

int jit_launch(void* handle, const float* const* ins, uint64_t outer, uint32_t nk, uint64_t inner, float init,
               const float* caps16, float* out, float* split_scratch_or_null, uint32_t splits, cudaStream_t s) {
  // splits: CTAs per row for the split path (1 = none); top bit set = take the split path even with 1
  JitChain* jc = static_cast<JitChain*>(handle);
  tcabk::Caps caps;
  for (int i = 0; i < 16; ++i) caps.c[i] = caps16[i];
  const float* ptrs[TCAB_MAX_INPUTS];  // Ptrs<NIN> is NIN pointers: a prefix of this array
  for (int i = 0; i < TCAB_MAX_INPUTS; ++i) ptrs[i] = ins[i < jc->n_in ? i : 0];
  bool al = true;
  for (int i = 0; i < jc->n_in; ++i) al = al && aligned16(ins[i]);
  if (inner == 1) {
    if (jc->cells) return fail(TCAB_ERR_UNSUPPORTED, "chain_reduce: the chain was prepared for a middle-axis reduction");
    const bool vec = al && (nk % 4 == 0);
    const uint32_t nvec = vec ? nk / 4 : nk;
    const bool force_split = (splits & 0x80000000u) != 0;  // the entry point that allocates nothing
    splits &= 0x7fffffffu;
    // every operand bf16 and rows of whole 16-byte vectors: vectors of eight (rows from 128 columns; shorter ones
    // keep the kernels for short rows below)
    const bool vec8 = vec && jc->all_bf16 && nk % 8 == 0 && nk >= 128 && jc->k[kInner32V8] != nullptr;
    if ((splits > 1 || force_split) && split_scratch_or_null != nullptr) {
      const uint32_t rows = static_cast<uint32_t>(outer);
      const uint32_t nv = vec8 && !force_split ? nk / 8 : nvec;
      uint32_t sp = splits > nv ? (nv ? nv : 1) : splits;
      uint32_t vec_per_split = (nv + sp - 1) / sp;
      void* a1[] = {ptrs, &split_scratch_or_null, &nk, &sp, &vec_per_split, &caps};
      int rc = launch(jc->k[vec8 && !force_split ? kSplitV8 : vec ? kSplitV4 : kSplitV1], static_cast<uint64_t>(rows) * sp, 256, a1, s,
                      "chain_inner_split");
      if (rc != TCAB_OK) return rc;
      return launch_jit_finish(jc, split_scratch_or_null, out, rows, sp, init, caps, s);
    }
    if (vec8 && tune(kReduceInner).p0 <= 0) {  // a warp or a CTA per row, the thresholds counted in 16-byte vectors
      const bool cta = nk / 8 >= inner_cta_per_row_from(jc->n_in);
      void* a8[] = {ptrs, &out, &outer, &nk, &init, &caps};
      if (nk / 8 <= 64) return launch(jc->k[kInner4V8], (outer + 31) / 32, 128, a8, s, "chain_inner");  // four threads per row
      return launch(jc->k[cta ? kInner256V8 : kInner32V8], cta ? outer : (outer + 3) / 4, cta ? 256 : 128, a8, s, "chain_inner");
    }
    if (vec && nvec >= 2 && nvec <= 16 && outer >= 1024 && jc->k[kInnerRows32] != nullptr && tune(kReduceInner).p0 <= 0 &&
        rows32_warps(nvec, jc->n_in) >= 2) {  // a thread per row over a coalesced copy (same policy as ahead of time)
      const uint32_t warps = rows32_warps(nvec, jc->n_in);
      uint32_t nv = nvec;
      void* af[] = {ptrs, &out, &outer, &nv, &init, &caps};
      return launch(jc->k[kInnerRows32], (outer + warps * 32ull - 1) / (warps * 32ull), 32 * warps, af, s, "chain_inner_rows32",
                    static_cast<size_t>(warps) * jc->n_in * 32 * (nvec + 1) * 16);
    }
    // rows that are not whole vectors on aligned operands (same policy as the ahead-of-time path)
    if (al && !vec && tune(kReduceInner).p0 <= 0 && jc->k[kInnerRows32e] != nullptr) {
      const uint32_t warps = rows32e_warps(nk, jc->n_in);
      void* af[] = {ptrs, &out, &outer, &nk, &init, &caps};
      if (nk <= 64 && outer >= 1024 && warps >= 1)
        return launch(jc->k[kInnerRows32e], (outer + warps * 32ull - 1) / (warps * 32ull), 32 * warps, af, s,
                      "chain_inner_rows32e", static_cast<size_t>(warps) * jc->n_in * 32 * nk * 4);
      if (nk > 64) {  // the thresholds of whole-vector rows
        if (nk / 4 <= 64) return launch(jc->k[kInnerRag4], (outer + 31) / 32, 128, af, s, "chain_inner");
        const bool cta = nk / 4 >= inner_cta_per_row_from(jc->n_in);
        return launch(jc->k[cta ? kInnerRag256 : kInnerRag32], cta ? outer : (outer + 3) / 4, cta ? 256 : 128, af, s, "chain_inner");
      }
    }
    if (vec && nvec >= 1 && (nvec <= 32 || (nvec > 48 && nvec <= 64)) && outer >= 1024 && jc->k[kInnerFlat] != nullptr &&
        tune(kReduceInner).p0 <= 0) {
      uint32_t g = 1, nv = nvec;  // short rows: lanes along the row (same policy as the ahead-of-time path)
      while (g < nvec && g < 32) g <<= 1;
      const uint64_t rows_per_cta = static_cast<uint64_t>(8) * 4 * (32 / g);
      void* af[] = {ptrs, &out, &outer, &nv, &g, &init, &caps};
      return launch(jc->k[nvec <= 32 ? kInnerFlat : kInnerFlat2], (outer + rows_per_cta - 1) / rows_per_cta,
                    256, af, s, "chain_inner_flat");
    }
    const int t = nvec <= 16 ? 0 : nvec <= 64 ? 1 : nvec < (vec ? inner_cta_per_row_from(jc->n_in) : 1024u) ? 2 : 3;  // the same thresholds as the ahead-of-time path
    const int tpr = t == 0 ? 1 : t == 1 ? 4 : t == 2 ? 32 : 256;
    const bool big = vec && t == 2 && inner_wants_big_ctas(outer);        // small problems: 1024-thread CTAs
    const int threads = big ? 1024 : tpr > 128 ? tpr : 128;
    const uint64_t groups = threads / tpr;
    void* a[] = {ptrs, &out, &outer, &nk, &init, &caps};
    return launch(big ? jc->k[kInner32V4Big] : jc->k[(vec ? kInner1V4 : kInner1V1) + t], (outer + groups - 1) / groups, threads, a,
                  s, "chain_inner");
  }
  if (inner > 0xffffffffull) return fail(TCAB_ERR_TOO_LARGE, "chain_reduce: inner extent beyond 2^32");
  if (jc->broadcast)
    return fail(TCAB_ERR_UNSUPPORTED, "chain_reduce: operands with broadcast extents are taken by innermost-axis reductions only");
  const bool vec = al && (inner % 4 == 0);
  uint32_t nb = static_cast<uint32_t>(outer), nc = static_cast<uint32_t>(inner);
  uint32_t tiles_per_b = (nc + (vec ? 128 : 32) - 1) / (vec ? 128 : 32);
  const uint64_t tiles = static_cast<uint64_t>(nb) * tiles_per_b;
  if (tiles > 0xffffffffull) return fail(TCAB_ERR_TOO_LARGE, "chain_reduce: too many column tiles");
  // narrow rows and short reduced axes: a warp per (b, column tile) (same policy as the ahead-of-time path)
  const cudaKernel_t flat = jc->k[vec ? kOuterFlat : kOuterFlat1];
  if (flat != nullptr && tune(kReduceInner).p3 <= 0) {
    const uint32_t g = tune(kReduceInner).p0 == 32 ? outer_flat_width(nc, vec) : outer_flat_groups(nb, nk, nc, sm_count(), vec);
    if (g != 0) {
      uint32_t tpb = (nc + (vec ? 128 : 32) - 1) / (vec ? 128 : 32);
      const uint64_t work = static_cast<uint64_t>(nb) * tpb;
      uint32_t klen = nk;
      uint32_t ksplit =
          split_scratch_or_null == nullptr ? 1u : outer_flat_ranges(nb, nk, nc, g, vec, sm_count(), 262144, &klen);
      if (ksplit == 1) klen = nk;
      void* af[] = {ptrs, &out, &nb, &nk, &nc, &tpb, const_cast<uint32_t*>(&g), &init, &caps, &ksplit, &klen, &split_scratch_or_null};
      // a CTA per range, or eight tiles per CTA
      int rc = launch(flat, ksplit > 1 ? work * ksplit : (work + 7) / 8, 256, af, s, "chain_outer_flat");
      if (rc != TCAB_OK || ksplit == 1) return rc;
      return launch_jit_finish(jc, split_scratch_or_null, out, nb * nc, ksplit, init, caps, s);
    }
  }
  // few column tiles and a long k: the k axis is split over CTAs too (same policy as the ahead-of-time path)
  // (vectors of eight for bf16 operands were measured here too: behind the 8-byte loads of this kernel on most shapes)
  const cudaKernel_t kern = jc->k[vec ? kOuterV4 : kOuterV1];
  const int occ = occupancy(reinterpret_cast<const void*>(kern), 256, 0);
  uint32_t ksplit = split_scratch_or_null == nullptr
                        ? 1u
                        : choose_outer_splits(tiles, static_cast<uint64_t>(nb) * nc, nk,
                                              static_cast<uint64_t>(occ > 0 ? occ : 1) * sm_count());
  uint32_t klen = nk;
  plan_outer_ranges(ksplit, nk, &ksplit, &klen);  // no range starts at or past nk
  void* a[] = {ptrs, &out, &nb, &nk, &nc, &tiles_per_b, &init, &caps, &ksplit, &klen, &split_scratch_or_null};
  int rc = launch(kern, tiles * ksplit, 256, a, s, "chain_outer");
  if (rc != TCAB_OK || ksplit == 1) return rc;
  return launch_jit_finish(jc, split_scratch_or_null, out, nb * nc, ksplit, init, caps, s);
}

int jit_launch_batched(void* handle, const float* const* ins, float* const* outs, uint32_t nprob, uint32_t rows, uint32_t nk,
                       float init, const float* caps16, cudaStream_t s) {
  JitChain* jc = static_cast<JitChain*>(handle);
  if (jc->kind != 'B') return fail(TCAB_ERR_INVALID_ARG, "chain_reduce_batched: the chain was prepared for another use");
  tcabk::Caps caps;
  for (int i = 0; i < 16; ++i) caps.c[i] = caps16[i];
  // BatchPtrs<NIN>: kMaxBatch rows of NIN input pointers, then kMaxBatch output pointers
  const void* flat[tcabk::kMaxBatch * TCAB_MAX_INPUTS + tcabk::kMaxBatch] = {};
  bool al = true;
  for (uint32_t b = 0; b < nprob; ++b)
    for (int i = 0; i < jc->n_in; ++i) {
      flat[b * jc->n_in + i] = ins[b * jc->n_in + i];
      al = al && aligned16(ins[b * jc->n_in + i]);
    }
  for (uint32_t b = 0; b < nprob; ++b) flat[tcabk::kMaxBatch * jc->n_in + b] = outs[b];
  const bool vec = al && (nk % 4 == 0);
  const uint32_t nvec = vec ? nk / 4 : nk;
  const bool cta_per_row = nvec >= 1024;
  const uint64_t total = static_cast<uint64_t>(nprob) * rows;
  void* a[] = {flat, &nprob, &rows, &nk, &init, &caps};
  return launch(jc->k[(vec ? kBatch32V4 : kBatch32V1) + (cta_per_row ? 1 : 0)], cta_per_row ? total : (total + 7) / 8, 256, a, s,
                "chain_inner_batched");
}

int jit_launch_map(void* handle, const void* const* ins, void* out, uint64_t n, uint32_t cols, const float* caps16,
                   cudaStream_t s) {
  JitChain* jc = static_cast<JitChain*>(handle);
  if (jc->kind != 'M') return fail(TCAB_ERR_INVALID_ARG, "map: the chain was prepared for another use");
  tcabk::Caps caps;
  for (int i = 0; i < 16; ++i) caps.c[i] = caps16[i];
  const void* ptrs[TCAB_MAX_INPUTS];
  for (int i = 0; i < TCAB_MAX_INPUTS; ++i) ptrs[i] = ins[i < jc->n_in ? i : 0];
  bool al = aligned16(out);
  for (int i = 0; i < jc->n_in; ++i) al = al && aligned16(ins[i]);
  void* a[] = {ptrs, &out, &n, &caps, &cols};
  // one more group index than groups: the thread that gets it takes the ragged end
  if (al) return launch(jc->k[kMap8], (n / 8 + 1 + 255) / 256, 256, a, s, "chain_map");
  return launch(jc->k[kMap1], (n + 255) / 256, 256, a, s, "chain_map");
}

int jit_launch_contract(void* handle, const float* lhs, const float* rhs, int rhs_nk, float* out, uint32_t m,
                        uint32_t n, uint32_t k, float init, const float* caps16, cudaStream_t s) {
  JitChain* jc = static_cast<JitChain*>(handle);
  if (jc->n_in != 2 || jc->kind != 'C')  // a handle prepared for reductions has no contraction kernels
    return fail(TCAB_ERR_INVALID_ARG, "chain_contract: the map lambda must take exactly two operands");
  tcabk::Caps caps;
  for (int i = 0; i < 16; ++i) caps.c[i] = caps16[i];
  void* a[] = {&lhs, &rhs, &out, &m, &n, &k, &init, &caps};
  const bool big = contract_big_tiles(m, n);
  const uint32_t tile = big ? 128 : 64;
  const int slot = big ? (rhs_nk ? kContractNK8 : kContractKN8) : (rhs_nk ? kContractNK : kContractKN);
  const cudaError_t e = cudaLaunchKernel(reinterpret_cast<const void*>(jc->k[slot]),
                                         dim3((n + tile - 1) / tile, (m + tile - 1) / tile), dim3(256), a, 0, s);
  count_launch();
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(TCAB_ERR_CUDA, "chain_contract: launch failed: %s", cudaGetErrorString(e));
  }
  return TCAB_OK;
}

}  // namespace tcab
