/*
 * Public C API of the i runtime, as exported by this repository's
 * libi_core.so.  Same 19 symbols, structs and calling convention as the
 * reference's core/i.h:8-70 (implemented there by core/src/lib.rs:61-334), so
 * a front-end written against the reference (ilang-python/ilang.py loads the
 * library named by ILANG_CORE_LIB, ilang.py:6-9) binds to this library
 * unchanged.
 *
 * Conventions (reference: core/src/lib.rs):
 *  - pointer-returning calls return NULL on error, int calls return -1 (0 = ok),
 *    i_exec returns {NULL, 0}, i_output_count returns 0; the message is read
 *    with i_error(), which is thread-local and valid until the next error on
 *    that thread (lib.rs:57-59, 326-334).
 *  - combinators copy their arguments; the caller frees both the arguments and
 *    the result (lib.rs:336-351).  Freeing NULL is a no-op (lib.rs:289-300).
 *  - tensors are dense row-major float32; `data` may be a host pointer (copied
 *    to the GPU and back inside the call) or a CUDA device pointer (used in
 *    place).  Inputs and outputs are borrowed for the duration of the call.
 *    i_exec_into runs on a stream of the library's own, which is ordered behind
 *    no stream of the caller: device operands must be complete when the call is
 *    made (synchronise the stream that produced them first); the call returns
 *    when the outputs are complete.  i_b200_exec_into (i_b200.h) takes the
 *    caller's stream instead and needs no such synchronisation.
 *  - i_exec_into and i_exec run on the GPU and fail with an i_error() message
 *    when no CUDA device is usable; there is no CPU fallback.
 */
#pragma once

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct i_component i_component;
typedef struct i_program i_program;

typedef struct {
  const float* data;
  const size_t* shape;
  size_t rank;
} i_tensor;

typedef struct {
  float* data;
  const size_t* shape;
  size_t rank;
} i_tensor_mut;

typedef struct {
  float* data;
  size_t* shape;
  size_t rank;
  size_t len;
} i_owned_tensor;

typedef struct {
  i_owned_tensor* tensors;
  size_t count;
} i_outputs;

/* core/i.h:32-38 — build components. */
i_component* i_parse(const char* src);
i_component* i_identity(void);
i_component* i_chain(const i_component* left, const i_component* right);
i_component* i_compose(const i_component* left, const i_component* right);
i_component* i_fanout(const i_component* left, const i_component* right);
i_component* i_pair(const i_component* left, const i_component* right);
i_component* i_swap(const i_component* component);

/* core/i.h:40-41 — i_code returns a description of the execution plan (the
 * reference returns generated C); i_compile recognises the graph and builds
 * the plan (the reference JIT-compiles C with cc, lib.rs:353-415). */
char* i_code(const i_component* component);
i_program* i_compile(const i_component* component);

/* core/i.h:43-50 — output arity, ranks and shapes for given inputs. */
size_t i_output_count(const i_program* program);
int i_output_ranks(const i_program* program, size_t* ranks);
int i_output_shapes(const i_program* program, const i_tensor* inputs, size_t input_count,
                    size_t** shapes);

/* core/i.h:52-64 — run. */
int i_exec_into(const i_program* program, const i_tensor* inputs, size_t input_count,
                i_tensor_mut* outputs, size_t output_count);
i_outputs i_exec(const i_program* program, const i_tensor* inputs, size_t input_count);

/* core/i.h:66-70 — errors and ownership. */
const char* i_error(void);
void i_component_free(i_component* component);
void i_program_free(i_program* program);
void i_outputs_free(i_outputs outputs);
void i_string_free(char* s);

#ifdef __cplusplus
}
#endif
