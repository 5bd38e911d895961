/*
 * lancet_raf_shim.h - C bridge to the RAF-style operator registry of the library.
 *
 * The operators of the hot path are C++ OpEnvs registered under the reference's dialect-qualified
 * names (raf.op.cuda.moe_encode, ..., raf.op.nccl._all_to_all, raf.op.cuda.lans); a C++ host uses
 * raf_shim::Dispatch directly (csrc/raf_shim/raf_shim.h).  These entry points let a host without
 * C++ (the Python tests) drive the same path: declare the outputs of a call, then dispatch and
 * execute it like RAF's interpreter does (src/impl/interpreter.cc:246-337 of the reference:
 * declare -> allocate outputs -> Dispatch -> satisfy requests -> Execute).
 *
 * A call's arguments are a flat array of values in schema order; a tuple is a LANCET_RAF_TUPLE
 * entry whose `ndim` is the number of fields, followed by the fields.
 */
#ifndef LANCET_RAF_SHIM_H_
#define LANCET_RAF_SHIM_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { LANCET_RAF_NONE = 0, LANCET_RAF_TENSOR = 1, LANCET_RAF_TUPLE = 2, LANCET_RAF_INT = 3, LANCET_RAF_FLOAT = 4 };

typedef struct {
  int kind;
  void* data;
  int dtype_code; /* 0 int, 1 uint, 2 float, 4 bfloat (DLPack codes) */
  int dtype_bits;
  int ndim; /* for a tuple: number of fields */
  int64_t shape[6];
  double scalar;
  int device_type; /* 1 cpu, 2 cuda */
} lancet_raf_value_t;

const char* lancet_raf_last_error(void);
/* Output tensors (flattened if a tuple) of `op` ("raf.op.moe_encode", ...) for these arguments. */
int lancet_raf_declare(const char* op, const lancet_raf_value_t* args, int n_values, lancet_raf_value_t* outs,
                       int max_outs, int* n_outs);
/* Dispatch through the dialect registry and execute on `stream` with the caller's output buffers;
 * workspaces are allocated and freed around the call; returns the dialect op that ran. */
int lancet_raf_execute(const char* op, const lancet_raf_value_t* args, int n_values, const lancet_raf_value_t* outs,
                       int n_outs, char* dialect_op, int dialect_op_len, void* stream);
/* Communicator handed to operators that issue RequestDistributed (a lancet_comm_t). */
int lancet_raf_set_communicator(void* comm, int rank, int size);
/* "dialect_op:plevel;..." in dispatch order; returns the number of entries. */
int lancet_raf_dialect_ops(const char* base_op, char* buf, int buf_len);

#ifdef __cplusplus
}
#endif
#endif /* LANCET_RAF_SHIM_H_ */
