/* tcab_host.h -- C ABI over the .tca text frontend (libtcab_host.so).
 *
 * The reference compiles a .tca module ahead of time: `tcacomp` parses it (internal/syntax/parser),
 * checks it (internal/syntax/semacheck), lowers it onto the pkg rungs (internal/syntax/build/build.go:27-36),
 * emits <name>.cu (internal/cg/cxx/emit.go:85-190) and the user calls the generated
 * <Name>Launch(tensors..., out, scalars..., stream) (internal/cg/cxx/launch.go:23-156).
 * Here the same text is parsed at run time and each kernel is launched by name on the kernels of libtcab.so:
 * tcab_module_parse replaces the compile step, tcab_module_launch replaces the generated launcher. Tensors
 * and scalar parameters are passed by the names the kernel's signature gives them; the output tensor goes
 * by the name of the returned `let`.
 *
 * Plain C: pointers, sizes and status codes (tcab_status of tcab.h). Handles are not thread-safe; distinct
 * handles may be used from distinct threads. Messages are thread-local.
 */
#ifndef TCAB_HOST_H_
#define TCAB_HOST_H_

#include "tcab.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tcab_module tcab_module;

/* Parses and lowers every kernel of `text`. On success *out owns the module (free it with
 * tcab_module_free). On failure returns TCAB_ERR_INVALID_ARG (syntax, semantic checks: the message is
 * "line:col: ...", like the reference's diagnostics) or TCAB_ERR_UNSUPPORTED (a construct the reference's
 * grammar has but this path does not evaluate) and *out is NULL. Needs no GPU. */
TCAB_API int tcab_module_parse(const char* text, tcab_module** out);
/* The same for a module spread over several files: paths[i] / texts[i] are the files, `root` names the entry file.
 * The reference's loader reads the include graph from disk (internal/syntax/module.go:3-31); this library does
 * no file I/O, the host hands the texts over. @include paths are relative to the including file, may not be
 * absolute nor leave its directory; a file reached twice merges once; a cycle is an error; an included file's
 * kernels follow the including file's own. */
TCAB_API int tcab_module_parse_files(const char* const* paths, const char* const* texts, uint32_t n_files,
                                     const char* root, tcab_module** out);
TCAB_API void tcab_module_free(tcab_module* m);

TCAB_API uint32_t tcab_module_kernel_count(const tcab_module* m);
/* The launcher name of kernel i: @name(cxx="...") when present, else the kernel identifier
 * (internal/cg/cxx/naming.go). NULL when i is out of range. The pointers live as long as the module. */
TCAB_API const char* tcab_module_kernel_name(const tcab_module* m, uint32_t i);
/* The name the output tensor is bound by: the returned `let`. */
TCAB_API const char* tcab_module_kernel_output(const tcab_module* m, uint32_t i);
/* Which entry point of tcab.h the kernel lowers to: "chain_reduce", "chain_contract", "gemm_bias_act", "map",
 * "softmax_rows" or "layernorm_rows"; a kernel of several let chains lists its launches joined by '+' (statement
 * groups that spell a whole row softmax or layer-norm count as the one launch that replaces them). NULL with a
 * message when a chain has no kernel class. */
TCAB_API const char* tcab_module_kernel_class(const tcab_module* m, uint32_t i);

/* What the kernel lowers to, as newline-separated key=value lines (the pointer lives as long as the module):
 * class, out, inputs (comma-separated tensor names in operand order), and for the chain classes map, combine,
 * post (canonical lambda text over p0.. and c0..: what tcab_chain_reduce / tcab_chain_contract receive), init,
 * captures (scalar parameter of each capture slot), axis (reduced position) or rhs_is_nk; for gemm_bias_act
 * a, b, bias, act; always scalars (the scalar parameters in declaration order). A kernel of several launches has
 * class, out, launches (their number) and the keys of every launch prefixed "launch<i>."; locals lists the
 * intermediates that need device memory from the caller (bound by name like every tensor), local.<name> gives
 * each one's element type and dims. NULL with a message when a chain has no kernel class. */
TCAB_API const char* tcab_module_kernel_describe(const tcab_module* m, uint32_t i);

/* The kernel's tensors and scalar parameters, one per line: "<name>=<elem>[<dim>,...]" (a symbolic dim by its name,
 * a constant one by its extent; " local" follows an intermediate between statements) and "<name>=<elem>" for a
 * scalar. With it a host sizes the locals from the extents of the tensors it binds. */
TCAB_API const char* tcab_module_kernel_signature(const tcab_module* m, uint32_t i);

/* Launches kernel `kernel` (its launcher name) asynchronously on `stream` (a cudaStream_t). Every tensor
 * parameter, the output and every local that tcab_module_kernel_describe lists must be bound in
 * tensor_names/tensors (the caller owns all device memory, intermediates included), every scalar parameter in
 * scalar_names/scalars. Shapes are checked the way the generated launcher checks them
 * (internal/cg/cxx/launch.go:82-121): one extent per symbolic dim, constant extents exact. */
TCAB_API int tcab_module_launch(const tcab_module* m, const char* kernel, const char* const* tensor_names,
                                const tcab_tensor* tensors, uint32_t n_tensors, const char* const* scalar_names,
                                const float* scalars, uint32_t n_scalars, void* stream);

/* Message of the last failure of a tcab_module_* call on this thread. */
TCAB_API const char* tcab_host_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* TCAB_HOST_H_ */
