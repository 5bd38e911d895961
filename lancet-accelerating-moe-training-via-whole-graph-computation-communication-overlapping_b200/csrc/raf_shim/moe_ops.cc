// OpEnvs of the MoE hot path, registered under the reference's dialect-qualified names so that a
// RAF-style executor finds them where it found the originals:
//   raf.op.cuda.{moe_encode, moe_decode, moe_encode_dx, moe_encode_dg, moe_decode_dx, moe_decode_dg, lans}
//     (src/op/dialect/cuda/moe.cc:411, :1152, :1224, :1310, :1394, :1480; cuda/lans.cc:176-177)
//   raf.op.nccl._all_to_all (src/op/dialect/nccl/nccl.cc:285-286)
//   raf.op.nccl._all_to_allv (nccl.cc:438-439)
//   raf.op.cublas.{matmul, matmul_nt, matmul_tn, dense, sparse_expert_matmul_nt} (src/op/dialect/cublas/matmul.cc:328-335:
//     the expert GEMMs and their gradients, here on tcgen05; matmul_tt is not on the path and is left to the next dialect)
// Constructors see the concrete shapes and issue their workspace / stream requests; Execute only
// calls the C ABI on the current stream.  Declarations restate src/op/declare/moe.cc:26-299,
// declare/optimizer.cc:46-63 and declare/collective_comm.cc:54-81.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>

#include "../../../include/lancet_b200.h"
#include "../../../include/lancet_raf_shim.h"
#include "raf_shim.h"

namespace raf_shim {
namespace {

int LancetDType(const DType& d) {
  if (d.code == kFloat && d.bits == 32) return LANCET_F32;
  if (d.code == kFloat && d.bits == 16) return LANCET_F16;
  if (d.code == kBFloat && d.bits == 16) return LANCET_BF16;
  throw Error("unsupported dtype (float32, float16, bfloat16 only)");
}

void Ok(int rc) {
  if (rc != LANCET_OK) throw Error(std::string("lancet_b200: ") + lancet_last_error());
}

const Tensor& TensorArg(const CallValues& cv, size_t i) {
  RAF_SHIM_CHECK(i < cv.args.size() && cv.args[i].kind == Value::kTensor, "argument " + std::to_string(i) + " must be a tensor");
  return cv.args[i].tensor;
}

Tensor Make(const Device& dev, DType dt, std::vector<int64_t> shape) {
  Tensor t;
  t.device = dev;
  t.dtype = dt;
  t.shape = std::move(shape);
  return t;
}

int Capacity(int64_t S, int64_t E, float cf) { return lancet_moe_capacity((int)S, (int)E, cf, 1); }

// ---------------------------------------------------------------- declarations
void MoeEncodeDeclare(CallValues* call) {
  const Tensor& data = TensorArg(*call, 0);
  const Tensor& gate = TensorArg(*call, 1);
  const Tensor& used = TensorArg(*call, 2);
  RAF_SHIM_CHECK(data.shape.size() == 2, "Input data should be 2-D.");
  RAF_SHIM_CHECK(gate.shape.size() == 2, "Input gate should be 2-D.");
  RAF_SHIM_CHECK(used.shape.size() == 1, "Input used_capacity should be 1-D.");
  RAF_SHIM_CHECK(data.shape[0] == gate.shape[0], "Input data and gate should have matching shape in dim 0.");
  const float cf = call->args.size() > 3 ? (float)call->args[3].f : 1.0f;
  const int64_t S = data.shape[0], M = data.shape[1], E = gate.shape[1];
  const int64_t C = Capacity(S, E, cf);
  call->out = Value::Tuple({Value::T(Make(data.device, {kFloat, 32}, {S})), Value::T(Make(data.device, {kInt, 32}, {2, S})),
                            Value::T(Make(data.device, {kInt, 32}, {E})), Value::T(Make(data.device, {kUInt, 64}, {E})),
                            Value::T(Make(data.device, data.dtype, {E, C, M}))});
  call->device = data.device;
}

void MoeDecodeDeclare(CallValues* call) {
  const Tensor& data = TensorArg(*call, 0);
  const Tensor& il = TensorArg(*call, 2);
  RAF_SHIM_CHECK(data.shape.size() == 3 && il.shape.size() == 2, "moe_decode: data must be 3-D, indices_locations 2-D");
  call->out = Value::T(Make(data.device, data.dtype, {il.shape[1], data.shape[2]}));
  call->device = data.device;
}

void MoeEncodeDxDeclare(CallValues* call) {
  const Tensor& dy = TensorArg(*call, 0);
  const Tensor& il = TensorArg(*call, 1);
  RAF_SHIM_CHECK(dy.shape.size() == 3 && il.shape.size() == 2, "moe_encode_dx: dy must be 3-D, indices_locations 2-D");
  call->out = Value::T(Make(dy.device, dy.dtype, {il.shape[1], dy.shape[2]}));
  call->device = dy.device;
}

void MoeEncodeDgDeclare(CallValues* call) {
  const Tensor& dy = TensorArg(*call, 0);
  const Tensor& il = TensorArg(*call, 1);
  RAF_SHIM_CHECK(call->args.size() > 2, "moe_encode_dg: n_experts is required");
  call->out = Value::T(Make(dy.device, dy.dtype, {il.shape[1], call->args[2].i}));
  call->device = dy.device;
}

void MoeDecodeDxDeclare(CallValues* call) {
  const Tensor& dy = TensorArg(*call, 0);
  RAF_SHIM_CHECK(call->args.size() > 4 && dy.shape.size() == 2, "moe_decode_dx: dy [S,M], gate, indices_locations, n_experts, capacity");
  call->out = Value::T(Make(dy.device, dy.dtype, {call->args[3].i, call->args[4].i, dy.shape[1]}));
  call->device = dy.device;
}

void MoeDecodeDgDeclare(CallValues* call) {
  const Tensor& dy = TensorArg(*call, 0);
  call->out = Value::T(Make(dy.device, dy.dtype, {dy.shape[0]}));
  call->device = dy.device;
}

void LansDeclare(CallValues* call) {
  RAF_SHIM_CHECK(!call->args.empty() && call->args[0].kind == Value::kTuple, "lans: tensor_list must be a tuple");
  RAF_SHIM_CHECK(call->args[0].fields.size() % 4 == 0, "lans: tensor_list must hold 4 lists of equal length");
  call->out = call->args[0];  // in place: the output tuple aliases the inputs (declare/optimizer.cc:46-63)
  if (!call->out.fields.empty()) call->device = call->out.fields[0].tensor.device;
}

void AllToAllDeclare(CallValues* call) {
  RAF_SHIM_CHECK(!call->args.empty() && call->args[0].kind == Value::kTuple && !call->args[0].fields.empty(),
                 "_all_to_all: x must be a non-empty tuple of tensors");
  const auto& f = call->args[0].fields;
  if (f.size() == 1) {
    call->out = Value::T(Make(f[0].tensor.device, f[0].tensor.dtype, f[0].tensor.shape));
  } else {
    std::vector<Value> outs;
    for (const Value& v : f) outs.push_back(Value::T(Make(v.tensor.device, v.tensor.dtype, v.tensor.shape)));
    call->out = Value::Tuple(outs);
  }
  call->device = f[0].tensor.device;
}

void MatmulNtDeclare(CallValues* call) {
  const Tensor& a = TensorArg(*call, 0);
  const Tensor& b = TensorArg(*call, 1);
  RAF_SHIM_CHECK(a.shape.size() == 2 && b.shape.size() == 2 && a.shape[1] == b.shape[1], "matmul_nt: a [n,k], b [m,k]");
  call->out = Value::T(Make(a.device, a.dtype, {a.shape[0], b.shape[0]}));
  call->device = a.device;
}


void MoeEncodeBprDeclare(CallValues* call) {
  const Tensor& data = TensorArg(*call, 0);
  const Tensor& gate = TensorArg(*call, 1);
  RAF_SHIM_CHECK(data.shape.size() == 2 && gate.shape.size() == 2, "Expected input data to be 2D.");
  RAF_SHIM_CHECK(data.shape[0] == gate.shape[0], "Input data and gate should have matching shape in dim 0.");
  const int64_t n = call->args.size() > 2 ? call->args[2].i : 1;
  const float cf = call->args.size() > 4 ? (float)call->args[4].f : 1.0f;
  RAF_SHIM_CHECK(n >= 1 && data.shape[0] % n == 0, "the batch must split evenly into n_partitions");
  const int64_t S = data.shape[0] / n, M = data.shape[1], E = gate.shape[1];
  const int64_t C = Capacity(S, E, cf);  // from the per-partition token count (cuda/moe.cc:433-438)
  call->out = Value::Tuple({Value::T(Make(data.device, {kFloat, 32}, {S})), Value::T(Make(data.device, {kInt, 32}, {2, S})),
                            Value::T(Make(data.device, {kInt, 32}, {E})), Value::T(Make(data.device, {kUInt, 64}, {E})),
                            Value::T(Make(data.device, data.dtype, {E, C, M}))});
  call->device = data.device;
}

void MoeMergeMasksDeclare(CallValues* call) {
  RAF_SHIM_CHECK(!call->args.empty() && call->args[0].kind == Value::kTuple && !call->args[0].fields.empty(),
                 "moe_merge_masks: indices_locations must be a non-empty tuple");
  const Tensor& m0 = call->args[0].fields[0].tensor;
  RAF_SHIM_CHECK(m0.shape.size() == 2, "Input indices_locations should be 2-D.");
  call->out = Value::T(Make(m0.device, {kInt, 32}, {2, m0.shape[1] * (int64_t)call->args[0].fields.size()}));
  call->device = m0.device;
}

void MoeRedispatchDeclare(CallValues* call) {
  RAF_SHIM_CHECK(call->args.size() >= 2 && call->args[0].kind == Value::kTuple && !call->args[0].fields.empty(),
                 "moe_redispatch: data must be a non-empty tuple");
  const Tensor& d0 = call->args[0].fields[0].tensor;
  RAF_SHIM_CHECK(d0.shape.size() == 3, "moe_redispatch: data should be 3-D.");
  // the reference's declaration hard-codes float32 here (declare/moe.cc:136) while its type relation keeps the
  // input dtype (ty/moe.cc:141); the input dtype is used
  call->out = Value::T(Make(d0.device, d0.dtype, d0.shape));
  call->device = d0.device;
}

void MoeRedispatchExpertInputDeclare(CallValues* call) {
  RAF_SHIM_CHECK(call->args.size() >= 4 && call->args[0].kind == Value::kTuple && !call->args[0].fields.empty(),
                 "moe_redispatch_expert_input: data must be a non-empty tuple");
  const Tensor& d0 = call->args[0].fields[0].tensor;
  RAF_SHIM_CHECK(d0.shape.size() == 3, "moe_redispatch_expert_input: data should be [C, G, M].");
  call->out = Value::T(Make(d0.device, d0.dtype, d0.shape));
  call->device = d0.device;
}

RAF_OP_DECLARE("raf.op.moe_encode_batch_prioritized", MoeEncodeBprDeclare);
RAF_OP_DECLARE("raf.op.moe_merge_masks", MoeMergeMasksDeclare);
RAF_OP_DECLARE("raf.op.moe_redispatch", MoeRedispatchDeclare);
RAF_OP_DECLARE("raf.op.moe_redispatch_expert_input", MoeRedispatchExpertInputDeclare);

RAF_OP_DECLARE("raf.op.moe_encode", MoeEncodeDeclare);
RAF_OP_DECLARE("raf.op.moe_decode", MoeDecodeDeclare);
RAF_OP_DECLARE("raf.op.moe_encode_dx", MoeEncodeDxDeclare);
RAF_OP_DECLARE("raf.op.moe_encode_dg", MoeEncodeDgDeclare);
RAF_OP_DECLARE("raf.op.moe_decode_dx", MoeDecodeDxDeclare);
RAF_OP_DECLARE("raf.op.moe_decode_dg", MoeDecodeDgDeclare);
RAF_OP_DECLARE("raf.op.lans", LansDeclare);
RAF_OP_DECLARE("raf.op._all_to_all", AllToAllDeclare);
RAF_OP_DECLARE("raf.op.matmul_nt", MatmulNtDeclare);
RAF_OP_DECLARE("raf.op.dense", MatmulNtDeclare);

void MatmulDeclare(CallValues* call) {
  const Tensor& a = TensorArg(*call, 0);
  const Tensor& b = TensorArg(*call, 1);
  RAF_SHIM_CHECK(a.shape.size() == 2 && b.shape.size() == 2 && a.shape[1] == b.shape[0], "matmul: a [n,k], b [k,m]");
  call->out = Value::T(Make(a.device, a.dtype, {a.shape[0], b.shape[1]}));
  call->device = a.device;
}
void MatmulTnDeclare(CallValues* call) {
  const Tensor& a = TensorArg(*call, 0);
  const Tensor& b = TensorArg(*call, 1);
  RAF_SHIM_CHECK(a.shape.size() == 2 && b.shape.size() == 2 && a.shape[0] == b.shape[0], "matmul_tn: a [k,n], b [k,m]");
  call->out = Value::T(Make(a.device, a.dtype, {a.shape[1], b.shape[1]}));
  call->device = a.device;
}
// src/op/declare/moe.cc:243-261
void SparseExpertMatmulNtDeclare(CallValues* call) {
  const Tensor& data = TensorArg(*call, 0);
  const Tensor& weight = TensorArg(*call, 1);
  const Tensor& nelem = TensorArg(*call, 2);
  RAF_SHIM_CHECK(data.shape.size() == 3, "Expected input data to be 3D.");
  RAF_SHIM_CHECK(weight.shape.size() == 2, "Expected input weight to be 2D.");
  RAF_SHIM_CHECK(nelem.shape.size() == 1, "Expected input nelements_per_gpu to be 1D.");
  const int64_t stride = call->args.size() > 4 ? call->args[4].i : 1;
  RAF_SHIM_CHECK(stride >= 1 && data.shape[1] == nelem.shape[0] / stride,
                 "Input data and nelements should have matching shape in dim 1 and 0 after stride.");
  RAF_SHIM_CHECK(weight.shape[1] == data.shape[2], "Input weight and data should have matching shapes in dim 1 and 2.");
  call->out = Value::T(Make(data.device, data.dtype, {data.shape[0], data.shape[1], weight.shape[0]}));
  call->device = data.device;
}
// src/op/declare/collective_comm.cc:84-128: (x, send_counts) -> (tensor like x, tensor like send_counts)
void AllToAllvDeclare(CallValues* call) {
  RAF_SHIM_CHECK(call->args.size() >= 2 && call->args[0].kind == Value::kTuple && call->args[0].fields.size() == 1 &&
                     call->args[1].kind == Value::kTuple && call->args[1].fields.size() == 1,
                 "AllToAllv currently only supports one input tensor and one send_counts tensor.");
  const Tensor& x = call->args[0].fields[0].tensor;
  const Tensor& sc = call->args[1].fields[0].tensor;
  call->out = Value::Tuple({Value::T(Make(x.device, x.dtype, x.shape)), Value::T(Make(sc.device, sc.dtype, sc.shape))});
  call->device = x.device;
}
RAF_OP_DECLARE("raf.op.matmul", MatmulDeclare);
RAF_OP_DECLARE("raf.op.matmul_tn", MatmulTnDeclare);
RAF_OP_DECLARE("raf.op.sparse_expert_matmul_nt", SparseExpertMatmulNtDeclare);
RAF_OP_DECLARE("raf.op._all_to_allv", AllToAllvDeclare);

// ---------------------------------------------------------------- op envs
class MoeEncode : public OpEnv {
 public:
  explicit MoeEncode(const CallValues& cv) {
    const Tensor& data = TensorArg(cv, 0);
    const Tensor& gate = TensorArg(cv, 1);
    S_ = (int)data.shape[0]; M_ = (int)data.shape[1]; E_ = (int)gate.shape[1];
    cf_ = cv.args.size() > 3 ? (float)cv.args[3].f : 1.0f;
    dtype_ = LancetDType(data.dtype);
    gate_dtype_ = LancetDType(gate.dtype);
    arg_indices = {0, 1, 2};  // data, gate, used_capacity
    ws_bytes_ = lancet_moe_gate_workspace_bytes(S_, E_, 1);
    RequestWorkspace(&ws_, cv.device, (int64_t)ws_bytes_);  // replaces the S*E one-hot workspace (cuda/moe.cc:133)
  }
  std::string name() const override { return "raf.op.cuda.moe_encode"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1], cv.args[2]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    RAF_SHIM_CHECK(out.kind == Value::kTuple && out.fields.size() == 5, "Expected output to be a 5-Tuple");
    const auto& o = out.fields;
    Ok(lancet_moe_encode(in[0].tensor.data, in[1].tensor.data, gate_dtype_, (const int32_t*)in[2].tensor.data, cf_, S_, M_, E_,
                         1, dtype_, o[0].tensor.data, LancetDType(o[0].tensor.dtype), (int32_t*)o[1].tensor.data,
                         (int32_t*)o[2].tensor.data, (uint64_t*)o[3].tensor.data, o[4].tensor.data, ws_, ws_bytes_, 0,
                         GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new MoeEncode(cv); }

 private:
  int S_, M_, E_, dtype_, gate_dtype_;
  float cf_;
  void* ws_ = nullptr;
  size_t ws_bytes_ = 0;
};
RAF_REGISTER_DIALECT_OP(cuda, moe_encode, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.moe_encode", MoeEncode::make);

class MoeDecode : public OpEnv {
 public:
  explicit MoeDecode(const CallValues& cv) {
    const Tensor& data = TensorArg(cv, 0);
    E_ = (int)data.shape[0]; C_ = (int)data.shape[1]; M_ = (int)data.shape[2];
    S_ = (int)TensorArg(cv, 2).shape[1];
    dtype_ = LancetDType(data.dtype);
    arg_indices = {0, 1, 2};
  }
  std::string name() const override { return "raf.op.cuda.moe_decode"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1], cv.args[2]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    Ok(lancet_moe_decode_fwd(in[1].tensor.data, LancetDType(in[1].tensor.dtype), (const int32_t*)in[2].tensor.data, 1,
                             in[0].tensor.data, out.tensor.data, S_, M_, C_, E_, dtype_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new MoeDecode(cv); }

 private:
  int S_, M_, C_, E_, dtype_;
};
RAF_REGISTER_DIALECT_OP(cuda, moe_decode, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.moe_decode", MoeDecode::make);

class MoeEncodeDx : public OpEnv {
 public:
  explicit MoeEncodeDx(const CallValues& cv) {
    const Tensor& dy = TensorArg(cv, 0);
    E_ = (int)dy.shape[0]; C_ = (int)dy.shape[1]; M_ = (int)dy.shape[2];
    S_ = (int)TensorArg(cv, 1).shape[1];
    dtype_ = LancetDType(dy.dtype);
    arg_indices = {0, 1};
  }
  std::string name() const override { return "raf.op.cuda.moe_encode_dx"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    Ok(lancet_moe_encode_bwd_data((const int32_t*)in[1].tensor.data, 1, in[0].tensor.data, out.tensor.data, S_, M_, C_, E_,
                                  dtype_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new MoeEncodeDx(cv); }

 private:
  int S_, M_, C_, E_, dtype_;
};
RAF_REGISTER_DIALECT_OP(cuda, moe_encode_dx, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.moe_encode_dx", MoeEncodeDx::make);

class MoeEncodeDg : public OpEnv {
 public:
  explicit MoeEncodeDg(const CallValues& cv) {
    S_ = (int)TensorArg(cv, 1).shape[1];
    E_ = (int)cv.args.at(2).i;
    dtype_ = LancetDType(TensorArg(cv, 0).dtype);
    arg_indices = {0, 1};
  }
  std::string name() const override { return "raf.op.cuda.moe_encode_dg"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    Ok(lancet_moe_encode_bwd_gate(in[0].tensor.data, dtype_, (const int32_t*)in[1].tensor.data, 1, nullptr, dtype_,
                                  out.tensor.data, S_, E_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new MoeEncodeDg(cv); }

 private:
  int S_, E_, dtype_;
};
RAF_REGISTER_DIALECT_OP(cuda, moe_encode_dg, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.moe_encode_dg", MoeEncodeDg::make);

class MoeDecodeDx : public OpEnv {
 public:
  explicit MoeDecodeDx(const CallValues& cv) {
    const Tensor& dy = TensorArg(cv, 0);
    S_ = (int)dy.shape[0]; M_ = (int)dy.shape[1];
    E_ = (int)cv.args.at(3).i; C_ = (int)cv.args.at(4).i;
    dtype_ = LancetDType(dy.dtype);
    arg_indices = {0, 1, 2};
  }
  std::string name() const override { return "raf.op.cuda.moe_decode_dx"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1], cv.args[2]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    Ok(lancet_moe_decode_bwd_data(in[1].tensor.data, LancetDType(in[1].tensor.dtype), (const int32_t*)in[2].tensor.data, 1,
                                  in[0].tensor.data, out.tensor.data, nullptr, S_, M_, C_, E_, dtype_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new MoeDecodeDx(cv); }

 private:
  int S_, M_, C_, E_, dtype_;
};
RAF_REGISTER_DIALECT_OP(cuda, moe_decode_dx, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.moe_decode_dx", MoeDecodeDx::make);

class MoeDecodeDg : public OpEnv {
 public:
  explicit MoeDecodeDg(const CallValues& cv) {
    const Tensor& dy = TensorArg(cv, 0);
    const Tensor& data = TensorArg(cv, 1);
    S_ = (int)dy.shape[0]; M_ = (int)dy.shape[1];
    E_ = (int)data.shape[0]; C_ = (int)data.shape[1];
    dtype_ = LancetDType(dy.dtype);
    arg_indices = {0, 1, 2};
  }
  std::string name() const override { return "raf.op.cuda.moe_decode_dg"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1], cv.args[2]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    Ok(lancet_moe_decode_bwd_gate((const int32_t*)in[2].tensor.data, 1, in[0].tensor.data, in[1].tensor.data, out.tensor.data,
                                  LancetDType(out.tensor.dtype), S_, M_, C_, E_, dtype_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new MoeDecodeDg(cv); }

 private:
  int S_, M_, C_, E_, dtype_;
};
RAF_REGISTER_DIALECT_OP(cuda, moe_decode_dg, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.moe_decode_dg", MoeDecodeDg::make);


// moe_encode_batch_prioritized(data, gate, n_partitions, partition_id, capacity_factor): def_schema.py:648-654
class MoeEncodeBatchPrioritized : public OpEnv {
 public:
  explicit MoeEncodeBatchPrioritized(const CallValues& cv) {
    const Tensor& data = TensorArg(cv, 0);
    const Tensor& gate = TensorArg(cv, 1);
    S_ = (int)data.shape[0]; M_ = (int)data.shape[1]; E_ = (int)gate.shape[1];
    n_ = cv.args.size() > 2 ? (int)cv.args[2].i : 1;
    pid_ = cv.args.size() > 3 ? (int)cv.args[3].i : 0;
    cf_ = cv.args.size() > 4 ? (float)cv.args[4].f : 1.0f;
    dtype_ = LancetDType(data.dtype);
    gate_dtype_ = LancetDType(gate.dtype);
    arg_indices = {0, 1};
    ws_bytes_ = lancet_moe_gate_bpr_workspace_bytes(S_, E_);
    RequestWorkspace(&ws_, cv.device, (int64_t)ws_bytes_);
  }
  std::string name() const override { return "raf.op.cuda.moe_encode_batch_prioritized"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    RAF_SHIM_CHECK(out.kind == Value::kTuple && out.fields.size() == 5, "Expected output to be a 5-Tuple");
    const auto& o = out.fields;
    Ok(lancet_moe_encode_bpr(in[0].tensor.data, in[1].tensor.data, gate_dtype_, n_, pid_, cf_, S_, M_, E_, dtype_, o[0].tensor.data,
                             LancetDType(o[0].tensor.dtype), (int32_t*)o[1].tensor.data, (int32_t*)o[2].tensor.data,
                             (uint64_t*)o[3].tensor.data, o[4].tensor.data, ws_, ws_bytes_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new MoeEncodeBatchPrioritized(cv); }

 private:
  int S_, M_, E_, n_, pid_, dtype_, gate_dtype_;
  float cf_;
  void* ws_ = nullptr;
  size_t ws_bytes_ = 0;
};
RAF_REGISTER_DIALECT_OP(cuda, moe_encode_batch_prioritized, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.moe_encode_batch_prioritized", MoeEncodeBatchPrioritized::make);

class MoeMergeMasks : public OpEnv {
 public:
  explicit MoeMergeMasks(const CallValues& cv) {
    n_ = (int)cv.args[0].fields.size();
    S_ = (int)cv.args[0].fields[0].tensor.shape[1];
    E_ = (int)cv.args.at(1).i;
    arg_indices = {0};
    ws_bytes_ = lancet_moe_partition_workspace_bytes(n_, E_);
    RequestWorkspace(&ws_, cv.device, (int64_t)ws_bytes_);  // replaces the pinned pointer table of cuda/moe.cc:755-789
  }
  std::string name() const override { return "raf.op.cuda.moe_merge_masks"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    std::vector<const int32_t*> p;
    for (const Value& v : in[0].fields) p.push_back((const int32_t*)v.tensor.data);
    Ok(lancet_moe_merge_masks(p.data(), n_, S_, E_, (int32_t*)out.tensor.data, ws_, ws_bytes_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new MoeMergeMasks(cv); }

 private:
  int n_, S_, E_;
  void* ws_ = nullptr;
  size_t ws_bytes_ = 0;
};
RAF_REGISTER_DIALECT_OP(cuda, moe_merge_masks, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.moe_merge_masks", MoeMergeMasks::make);

class MoeRedispatch : public OpEnv {
 public:
  explicit MoeRedispatch(const CallValues& cv) {
    const Tensor& d0 = cv.args[0].fields[0].tensor;
    n_ = (int)cv.args[0].fields.size();
    RAF_SHIM_CHECK(cv.args[1].fields.size() == (size_t)n_, "moe_redispatch: one indices_locations per data tensor");
    E_ = (int)d0.shape[0]; C_ = (int)d0.shape[1]; M_ = (int)d0.shape[2];
    S_ = (int)cv.args[1].fields[0].tensor.shape[1];
    dtype_ = LancetDType(d0.dtype);
    arg_indices = {0, 1};
    ws_bytes_ = lancet_moe_partition_workspace_bytes(n_, E_);
    RequestWorkspace(&ws_, cv.device, (int64_t)ws_bytes_);
  }
  std::string name() const override { return "raf.op.cuda.moe_redispatch"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    std::vector<const void*> d;
    std::vector<const int32_t*> il;
    for (const Value& v : in[0].fields) d.push_back(v.tensor.data);
    for (const Value& v : in[1].fields) il.push_back((const int32_t*)v.tensor.data);
    Ok(lancet_moe_redispatch(d.data(), il.data(), n_, S_, M_, C_, E_, dtype_, out.tensor.data, ws_, ws_bytes_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new MoeRedispatch(cv); }

 private:
  int n_, S_, M_, C_, E_, dtype_;
  void* ws_ = nullptr;
  size_t ws_bytes_ = 0;
};
RAF_REGISTER_DIALECT_OP(cuda, moe_redispatch, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.moe_redispatch", MoeRedispatch::make);

// moe_redispatch_expert_input(data, recv_cnts, local_expert_id, n_local_experts, recv_cnts_scale): def_schema.py:670-684
class MoeRedispatchExpertInput : public OpEnv {
 public:
  explicit MoeRedispatchExpertInput(const CallValues& cv) {
    const Tensor& d0 = cv.args[0].fields[0].tensor;
    n_ = (int)cv.args[0].fields.size();
    RAF_SHIM_CHECK(cv.args[1].fields.size() == (size_t)n_, "moe_redispatch_expert_input: one recv_cnts per data tensor");
    C_ = (int)d0.shape[0]; G_ = (int)d0.shape[1]; M_ = (int)d0.shape[2];
    le_ = (int)cv.args.at(2).i; LE_ = (int)cv.args.at(3).i;
    scale_ = cv.args.size() > 4 ? (int)cv.args[4].i : 1;
    dtype_ = LancetDType(d0.dtype);
    arg_indices = {0, 1};
  }
  std::string name() const override { return "raf.op.cuda.moe_redispatch_expert_input"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    std::vector<const void*> d;
    std::vector<const uint64_t*> rc;
    for (const Value& v : in[0].fields) d.push_back(v.tensor.data);
    for (const Value& v : in[1].fields) rc.push_back((const uint64_t*)v.tensor.data);
    Ok(lancet_moe_redispatch_expert_input(d.data(), rc.data(), n_, le_, LE_, C_, G_, M_, scale_, dtype_, out.tensor.data, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new MoeRedispatchExpertInput(cv); }

 private:
  int n_, C_, G_, M_, le_, LE_, scale_, dtype_;
};
RAF_REGISTER_DIALECT_OP(cuda, moe_redispatch_expert_input, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.moe_redispatch_expert_input", MoeRedispatchExpertInput::make);

// lans(tensor_list = g + x + m + v, step, learning_rate, beta1, beta2, eps, bias_correction, weight_decay,
//      grad_averaging, mode, normalize_grad): scripts/src_codegen/def_schema.py:726-742, cuda/lans.cc:26-177
class LansImpl : public OpEnv {
 public:
  explicit LansImpl(const CallValues& cv) {
    RAF_SHIM_CHECK(cv.args.size() >= 11, "lans takes 11 arguments");
    const auto& tl = cv.args[0].fields;
    RAF_SHIM_CHECK(tl.size() % 4 == 0, "lans: tensor_list must hold 4 lists of equal length");
    n_ = (int)tl.size() / 4;
    for (int i = 0; i < n_; ++i) {
      RAF_SHIM_CHECK(tl[i].tensor.dtype.code == kFloat && tl[i].tensor.dtype.bits == 32, "Unsupported dtype: only float32");
      numels_.push_back(tl[i].tensor.numel());
    }
    lr_ = (float)cv.args[2].f; beta1_ = (float)cv.args[3].f; beta2_ = (float)cv.args[4].f; eps_ = (float)cv.args[5].f;
    bias_correction_ = (int)cv.args[6].i; wd_ = (float)cv.args[7].f; grad_averaging_ = (int)cv.args[8].i;
    mode_ = (int)cv.args[9].i; normalize_grad_ = cv.args[10].i != 0;
    arg_indices = {0, 1};
    ws_bytes_ = n_ ? lancet_lans_workspace_bytes(n_, numels_.data()) : 0;
    if (ws_bytes_) RequestWorkspace(&ws_, cv.device, (int64_t)ws_bytes_);
  }
  std::string name() const override { return "raf.op.cuda.lans"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value /*output aliases the inputs*/) override {
    if (n_ == 0) return;
    const auto& tl = in[0].fields;
    std::vector<void*> g(n_), p(n_), m(n_), v(n_);
    for (int i = 0; i < n_; ++i) {
      g[i] = tl[i].tensor.data; p[i] = tl[n_ + i].tensor.data; m[i] = tl[2 * n_ + i].tensor.data; v[i] = tl[3 * n_ + i].tensor.data;
    }
    // The workspace belongs to the executor, which may hand the same address out again after another op has used
    // it as scratch (src/impl/vm/vm.cc:1260-1266, interpreter.cc:283-323): nothing is kept in it between calls, the
    // tensor table and the counters are written on every call (one small copy and two memsets on the stream).
    const int flags = 0;
    const Value& s = in[1];
    if (s.kind == Value::kTensor && s.tensor.device.device_type != 1) {
      // step as the reference passes it, a device scalar (cuda/lans.cc:102-107): it stays on the device, no read-back
      Ok(lancet_lans_dev_step(ws_, ws_bytes_, n_, numels_.data(), g.data(), p.data(), m.data(), v.data(), LANCET_F32,
                              static_cast<const float*>(s.tensor.data), lr_, beta1_, beta2_, eps_, bias_correction_, wd_,
                              grad_averaging_, mode_, normalize_grad_ ? 1 : 0, flags, GetStream()));
      return;
    }
    const float fstep = s.kind == Value::kTensor ? *static_cast<const float*>(s.tensor.data) : (float)s.f;
    Ok(lancet_lans(ws_, ws_bytes_, n_, numels_.data(), g.data(), p.data(), m.data(), v.data(), LANCET_F32, (int)fstep, lr_, beta1_,
                   beta2_, eps_, bias_correction_, wd_, grad_averaging_, mode_, normalize_grad_ ? 1 : 0, flags, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) { return new LansImpl(cv); }

 private:
  int n_ = 0, bias_correction_ = 1, grad_averaging_ = 1, mode_ = 1;
  bool normalize_grad_ = true;
  float lr_, beta1_, beta2_, eps_, wd_;
  std::vector<int64_t> numels_;
  void* ws_ = nullptr;
  size_t ws_bytes_ = 0;
};
RAF_REGISTER_DIALECT_OP(cuda, lans, 20);
RAF_OP_ENV_MAKER("raf.op.cuda.lans", LansImpl::make);

// _all_to_all over NCCL: one tensor directly, a tuple through pack / one exchange / unpack (nccl.cc:195-277)
class NCCLAllToAll : public OpEnv {
 public:
  explicit NCCLAllToAll(const CallValues& cv) {
    arg_indices = {0};
    RequestStream(&stream_, cv.device, kCudaCommunicate);
    RequestDistributed(&communicator_);
    for (const Value& v : cv.args[0].fields) {
      sizes_.push_back((size_t)v.tensor.nbytes());
      total_bytes_ += (size_t)v.tensor.nbytes();
    }
    if (sizes_.size() > 1) {
      RequestWorkspace(&in_ws_, cv.device, (int64_t)total_bytes_);
      RequestWorkspace(&out_ws_, cv.device, (int64_t)total_bytes_);
    }
  }
  std::string name() const override { return "raf.op.nccl._all_to_all"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    RAF_SHIM_CHECK(communicator_ != nullptr, "_all_to_all: no communicator (RequestDistributed was not satisfied)");
    if (sizes_.size() == 1) {
      // the world size is the communicator's; the split must be even (nccl.cc:213)
      Ok(lancet_all_to_all_evenly(in[0].fields[0].tensor.data, out.tensor.data, total_bytes_, communicator_, stream_));
      return;
    }
    std::vector<const void*> s;
    std::vector<void*> r;
    for (const Value& v : in[0].fields) s.push_back(v.tensor.data);
    for (const Value& v : out.fields) r.push_back(v.tensor.data);
    Ok(lancet_all_to_all_tuple(s.data(), r.data(), sizes_.data(), (int)sizes_.size(), in_ws_, out_ws_, total_bytes_, communicator_,
                               stream_));
  }
  static OpEnv* make(const CallValues& cv) {
    if (cv.args.empty() || cv.args[0].kind != Value::kTuple || cv.args[0].fields.empty() || cv.args[0].fields.size() > 16)
      return nullptr;
    return new NCCLAllToAll(cv);
  }

 private:
  void* stream_ = nullptr;
  void* communicator_ = nullptr;
  void* in_ws_ = nullptr;
  void* out_ws_ = nullptr;
  std::vector<size_t> sizes_;
  size_t total_bytes_ = 0;
};
RAF_REGISTER_DIALECT_OP(nccl, _all_to_all, 10);
RAF_OP_ENV_MAKER("raf.op.nccl._all_to_all", NCCLAllToAll::make);

// matmul_nt(a [n,k], b [m,k]) -> [n,m]: the expert GEMM as one group on the tcgen05 kernel.  Declines
// shapes or types the kernel does not take (the dispatcher then tries the next dialect).
class MatmulNt : public OpEnv {
 public:
  explicit MatmulNt(const CallValues& cv) {
    const Tensor& a = TensorArg(cv, 0);
    const Tensor& b = TensorArg(cv, 1);
    n_ = (int)a.shape[0]; k_ = (int)a.shape[1]; m_ = (int)b.shape[0];
    dtype_ = LancetDType(a.dtype);
    arg_indices = {0, 1};
    RequestWorkspace(&status_, cv.device, 256);
  }
  std::string name() const override { return "raf.op.cublas.matmul_nt"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    RAF_SHIM_CHECK(cudaMemsetAsync(status_, 0, 4, (cudaStream_t)GetStream()) == cudaSuccess, "memset failed");
    Ok(lancet_grouped_gemm_nt(in[0].tensor.data, in[1].tensor.data, out.tensor.data, nullptr, nullptr, 1, 1, n_, m_, k_, nullptr, 0,
                              dtype_, (int32_t*)status_, GetStream()));
  }
  static bool Accepts(const CallValues& cv) {
    if (cv.args.size() < 2 || cv.args[0].kind != Value::kTensor || cv.args[1].kind != Value::kTensor) return false;
    const Tensor& a = cv.args[0].tensor;
    const Tensor& b = cv.args[1].tensor;
    if (a.dtype.bits != 16 || !(a.dtype == b.dtype)) return false;
    return a.shape.size() == 2 && b.shape.size() == 2 && b.shape[0] % 256 == 0 && a.shape[1] % 8 == 0;
  }
  static OpEnv* make(const CallValues& cv) { return Accepts(cv) ? new MatmulNt(cv) : nullptr; }

 protected:
  int n_, k_, m_, dtype_;
  void* status_ = nullptr;
};
RAF_REGISTER_DIALECT_OP(cublas, matmul_nt, 15);
RAF_OP_ENV_MAKER("raf.op.cublas.matmul_nt", MatmulNt::make);

// dense(x [n,k], w [m,k]) is the same contraction under another name (nn.Linear without bias)
class Dense : public MatmulNt {
 public:
  using MatmulNt::MatmulNt;
  std::string name() const override { return "raf.op.cublas.dense"; }
  static OpEnv* make(const CallValues& cv) { return Accepts(cv) ? new Dense(cv) : nullptr; }
};
RAF_REGISTER_DIALECT_OP(cublas, dense, 15);
RAF_OP_ENV_MAKER("raf.op.cublas.dense", Dense::make);

// matmul(a [n,k], b [k,m]) -> [n,m]: the data-gradient form (dX = matmul(dy, w), src/op/grad/gemm.cc:31-36)
class Matmul : public OpEnv {
 public:
  explicit Matmul(const CallValues& cv) {
    const Tensor& a = TensorArg(cv, 0);
    const Tensor& b = TensorArg(cv, 1);
    n_ = (int)a.shape[0]; k_ = (int)a.shape[1]; m_ = (int)b.shape[1];
    dtype_ = LancetDType(a.dtype);
    arg_indices = {0, 1};
    RequestWorkspace(&status_, cv.device, 256);
  }
  std::string name() const override { return "raf.op.cublas.matmul"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    RAF_SHIM_CHECK(cudaMemsetAsync(status_, 0, 4, (cudaStream_t)GetStream()) == cudaSuccess, "memset failed");
    Ok(lancet_grouped_gemm_nn(in[0].tensor.data, in[1].tensor.data, out.tensor.data, nullptr, 1, 1, n_, m_, k_, nullptr, 0, dtype_,
                              (int32_t*)status_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) {
    if (cv.args.size() < 2 || cv.args[0].kind != Value::kTensor || cv.args[1].kind != Value::kTensor) return nullptr;
    const Tensor& a = cv.args[0].tensor;
    const Tensor& b = cv.args[1].tensor;
    if (a.dtype.bits != 16 || !(a.dtype == b.dtype)) return nullptr;
    if (a.shape.size() != 2 || b.shape.size() != 2 || b.shape[1] % 256 != 0 || a.shape[1] % 64 != 0) return nullptr;
    return new Matmul(cv);
  }

 private:
  int n_, k_, m_, dtype_;
  void* status_ = nullptr;
};
RAF_REGISTER_DIALECT_OP(cublas, matmul, 15);
RAF_OP_ENV_MAKER("raf.op.cublas.matmul", Matmul::make);

// matmul_tn(a [k,n], b [k,m]) -> [n,m]: the weight-gradient form (dW = matmul_tn(dy, x), src/op/grad/gemm.cc:31-36)
class MatmulTn : public OpEnv {
 public:
  explicit MatmulTn(const CallValues& cv) {
    const Tensor& a = TensorArg(cv, 0);
    const Tensor& b = TensorArg(cv, 1);
    k_ = (int)a.shape[0]; n_ = (int)a.shape[1]; m_ = (int)b.shape[1];
    dtype_ = LancetDType(a.dtype);
    arg_indices = {0, 1};
    RequestWorkspace(&status_, cv.device, 256);
  }
  std::string name() const override { return "raf.op.cublas.matmul_tn"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    RAF_SHIM_CHECK(cudaMemsetAsync(status_, 0, 4, (cudaStream_t)GetStream()) == cudaSuccess, "memset failed");
    Ok(lancet_grouped_gemm_tn(in[0].tensor.data, in[1].tensor.data, out.tensor.data, 1, 1, k_, n_, m_, nullptr, dtype_,
                              (int32_t*)status_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) {
    if (cv.args.size() < 2 || cv.args[0].kind != Value::kTensor || cv.args[1].kind != Value::kTensor) return nullptr;
    const Tensor& a = cv.args[0].tensor;
    const Tensor& b = cv.args[1].tensor;
    if (a.dtype.bits != 16 || !(a.dtype == b.dtype)) return nullptr;
    if (a.shape.size() != 2 || b.shape.size() != 2 || a.shape[1] % 128 != 0 || b.shape[1] % 256 != 0) return nullptr;
    return new MatmulTn(cv);
  }

 private:
  int n_, k_, m_, dtype_;
  void* status_ = nullptr;
};
RAF_REGISTER_DIALECT_OP(cublas, matmul_tn, 15);
RAF_OP_ENV_MAKER("raf.op.cublas.matmul_tn", MatmulTn::make);

// sparse_expert_matmul_nt(data [C,G,M], weight [N,M], nelements_per_gpu u64, offset, stride, scale) -> [C,G,N]
// (src/op/dialect/cublas/matmul.cc:144-326).  Only the rows each source rank really sent are multiplied (what the
// reference's commented-out path intended); the other rows of the output are zero.
class SparseExpertMatmulNt : public OpEnv {
 public:
  explicit SparseExpertMatmulNt(const CallValues& cv) {
    const Tensor& data = TensorArg(cv, 0);
    const Tensor& weight = TensorArg(cv, 1);
    C_ = (int)data.shape[0]; G_ = (int)data.shape[1]; M_ = (int)data.shape[2]; N_ = (int)weight.shape[0];
    offset_ = cv.args.size() > 3 ? (int)cv.args[3].i : 0;
    stride_ = cv.args.size() > 4 ? (int)cv.args[4].i : 1;
    scale_ = cv.args.size() > 5 ? (int)cv.args[5].i : 1;
    dtype_ = LancetDType(data.dtype);
    arg_indices = {0, 1, 2};
    ws_bytes_ = lancet_sparse_expert_matmul_nt_workspace_bytes(G_);
    RequestWorkspace(&ws_, cv.device, (int64_t)ws_bytes_);  // replaces the two input-sized scratch buffers (matmul.cc:189-190)
  }
  std::string name() const override { return "raf.op.cublas.sparse_expert_matmul_nt"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1], cv.args[2]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    Ok(lancet_sparse_expert_matmul_nt(in[0].tensor.data, in[1].tensor.data, out.tensor.data, (const uint64_t*)in[2].tensor.data,
                                      offset_, stride_, scale_, C_, G_, M_, N_, dtype_, ws_, ws_bytes_, GetStream()));
  }
  static OpEnv* make(const CallValues& cv) {
    if (cv.args.size() < 3 || cv.args[0].kind != Value::kTensor || cv.args[1].kind != Value::kTensor ||
        cv.args[2].kind != Value::kTensor)
      return nullptr;
    const Tensor& d = cv.args[0].tensor;
    const Tensor& w = cv.args[1].tensor;
    if (d.dtype.bits != 16 || !(d.dtype == w.dtype) || cv.args[2].tensor.dtype.bits != 64) return nullptr;
    if (d.shape.size() != 3 || w.shape.size() != 2 || w.shape[0] % 256 != 0 || d.shape[2] % 8 != 0) return nullptr;
    return new SparseExpertMatmulNt(cv);
  }

 private:
  int C_, G_, M_, N_, offset_, stride_, scale_, dtype_;
  void* ws_ = nullptr;
  size_t ws_bytes_ = 0;
};
RAF_REGISTER_DIALECT_OP(cublas, sparse_expert_matmul_nt, 20);
RAF_OP_ENV_MAKER("raf.op.cublas.sparse_expert_matmul_nt", SparseExpertMatmulNt::make);

// _all_to_allv over NCCL (nccl.cc:288-439) without the reference's device-to-host copy of the counts and stream
// synchronisation (:388-390): the counts are exchanged on the device, whole chunks travel, and a kernel clears what
// lies past the received counts.
class NCCLAllToAllv : public OpEnv {
 public:
  explicit NCCLAllToAllv(const CallValues& cv) {
    arg_indices = {0, 1};
    RequestStream(&stream_, cv.device, kCudaCommunicate);
    RequestDistributed(&communicator_);
    const Tensor& x = cv.args[0].fields[0].tensor;
    const Tensor& sc = cv.args[1].fields[0].tensor;
    const int world = GetCommunicatorSize();
    RAF_SHIM_CHECK(world >= 1 && sc.numel() % world == 0, "send_counts must hold world_size * n_chunks entries");
    n_chunks_ = (int)(sc.numel() / world);
    RAF_SHIM_CHECK(n_chunks_ >= 1 && x.numel() % ((int64_t)world * n_chunks_) == 0,
                   "Cannot evenly distribute input tensor to all ranks and chunks.");
    chunk_elems_ = (size_t)(x.numel() / ((int64_t)world * n_chunks_));
    elem_size_ = (size_t)(x.dtype.bits / 8);
  }
  std::string name() const override { return "raf.op.nccl._all_to_allv"; }
  void Execute(const CallValues& cv) override { Execute({cv.args[0], cv.args[1]}, cv.out); }
  void Execute(const std::vector<Value>& in, Value out) override {
    RAF_SHIM_CHECK(communicator_ != nullptr, "_all_to_allv: no communicator (RequestDistributed was not satisfied)");
    RAF_SHIM_CHECK(out.kind == Value::kTuple && out.fields.size() == 2, "Expected output to be a 2-Tuple");
    Ok(lancet_all_to_allv(in[0].fields[0].tensor.data, out.fields[0].tensor.data, (const uint64_t*)in[1].fields[0].tensor.data,
                          (uint64_t*)out.fields[1].tensor.data, n_chunks_, elem_size_, chunk_elems_, communicator_, stream_));
  }
  static OpEnv* make(const CallValues& cv) {
    if (cv.args.size() < 2 || cv.args[0].kind != Value::kTuple || cv.args[0].fields.size() != 1 ||
        cv.args[1].kind != Value::kTuple || cv.args[1].fields.size() != 1)
      return nullptr;
    if (cv.args[1].fields[0].tensor.dtype.bits != 64) return nullptr;
    return new NCCLAllToAllv(cv);
  }

 private:
  void* stream_ = nullptr;
  void* communicator_ = nullptr;
  int n_chunks_ = 1;
  size_t chunk_elems_ = 0, elem_size_ = 1;
};
RAF_REGISTER_DIALECT_OP(nccl, _all_to_allv, 10);
RAF_OP_ENV_MAKER("raf.op.nccl._all_to_allv", NCCLAllToAllv::make);

// ---------------------------------------------------------------- C bridge for hosts without C++ (tests)
Value FromC(const lancet_raf_value_t* a, int n, int* pos) {
  const lancet_raf_value_t& v = a[(*pos)++];
  if (v.kind == LANCET_RAF_TENSOR) {
    Tensor t;
    t.data = v.data;
    t.device.device_type = v.device_type ? v.device_type : 2;
    t.dtype = {v.dtype_code, v.dtype_bits};
    t.shape.assign(v.shape, v.shape + v.ndim);
    return Value::T(t);
  }
  if (v.kind == LANCET_RAF_TUPLE) {
    std::vector<Value> f;
    for (int i = 0; i < v.ndim && *pos < n; ++i) f.push_back(FromC(a, n, pos));
    return Value::Tuple(f);
  }
  if (v.kind == LANCET_RAF_INT) return Value::Int((int64_t)v.scalar);
  if (v.kind == LANCET_RAF_FLOAT) return Value::Float(v.scalar);
  return Value();
}

void ToC(const Value& v, lancet_raf_value_t* outs, int max_outs, int* n) {
  if (v.kind == Value::kTuple) {
    for (const Value& f : v.fields) ToC(f, outs, max_outs, n);
    return;
  }
  if (v.kind != Value::kTensor) return;
  RAF_SHIM_CHECK(*n < max_outs, "too many outputs");
  lancet_raf_value_t& o = outs[(*n)++];
  std::memset(&o, 0, sizeof(o));
  o.kind = LANCET_RAF_TENSOR;
  o.data = v.tensor.data;
  o.dtype_code = v.tensor.dtype.code;
  o.dtype_bits = v.tensor.dtype.bits;
  o.device_type = v.tensor.device.device_type;
  RAF_SHIM_CHECK(v.tensor.shape.size() <= 6, "rank above 6");
  o.ndim = (int)v.tensor.shape.size();
  for (int i = 0; i < o.ndim; ++i) o.shape[i] = v.tensor.shape[i];
}

thread_local std::string g_err;

CallValues BuildCall(const char* op, const lancet_raf_value_t* args, int n_values) {
  CallValues cv;
  cv.op = op;
  int pos = 0;
  while (pos < n_values) cv.args.push_back(FromC(args, n_values, &pos));
  return cv;
}

}  // namespace
}  // namespace raf_shim

extern "C" {
using namespace raf_shim;

const char* lancet_raf_last_error(void) { return g_err.c_str(); }

int lancet_raf_declare(const char* op, const lancet_raf_value_t* args, int n_values, lancet_raf_value_t* outs, int max_outs,
                       int* n_outs) {
  try {
    CallValues cv = BuildCall(op, args, n_values);
    Declare(&cv);
    int n = 0;
    ToC(cv.out, outs, max_outs, &n);
    *n_outs = n;
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  }
}

int lancet_raf_execute(const char* op, const lancet_raf_value_t* args, int n_values, const lancet_raf_value_t* outs, int n_outs,
                       char* dialect_op, int dialect_op_len, void* stream) {
  std::vector<void*> workspaces;
  try {
    CallValues cv = BuildCall(op, args, n_values);
    Declare(&cv);
    // bind the caller's output buffers (the executor allocates them from the declaration)
    int k = 0;
    std::function<void(Value&)> bind = [&](Value& v) {
      if (v.kind == Value::kTuple) {
        for (Value& f : v.fields) bind(f);
      } else if (v.kind == Value::kTensor) {
        RAF_SHIM_CHECK(k < n_outs, "not enough output buffers");
        if (cv.op != "raf.op.lans") v.tensor.data = outs[k].data;
        ++k;
      }
    };
    bind(cv.out);
    SetStream(stream);
    std::shared_ptr<OpEnv> env = Dispatch(cv);
    if (dialect_op && dialect_op_len > 0) {
      std::strncpy(dialect_op, env->name().c_str(), dialect_op_len - 1);
      dialect_op[dialect_op_len - 1] = 0;
    }
    // what an executor does before Execute: satisfy the requests (src/impl/vm/vm.cc:1237-1266)
    const Requests& rq = env->GetRequests();
    for (const auto& w : rq.workspace) {
      void* p = nullptr;
      RAF_SHIM_CHECK(cudaMalloc(&p, (size_t)(w.nbytes > 0 ? w.nbytes : 1)) == cudaSuccess, "workspace allocation failed");
      workspaces.push_back(p);
      *w.dest = p;
    }
    for (const auto& s : rq.stream) *s.dest = stream;
    for (const auto& d : rq.distributed) *d.dest = GetCommunicator();
    env->Execute(cv);
    RAF_SHIM_CHECK(cudaStreamSynchronize((cudaStream_t)stream) == cudaSuccess, "stream synchronisation failed");
    for (void* p : workspaces) cudaFree(p);
    return 0;
  } catch (const std::exception& e) {
    for (void* p : workspaces) cudaFree(p);
    g_err = e.what();
    return 1;
  }
}

int lancet_raf_set_communicator(void* comm, int rank, int size) {
  SetCommunicator(comm, rank, size);
  return 0;
}

int lancet_raf_dialect_ops(const char* base_op, char* buf, int buf_len) {
  std::string s;
  for (const DialectEntry& e : DialectOps(base_op)) s += e.dialect_op + ":" + std::to_string(e.plevel) + ";";
  if (buf && buf_len > 0) {
    std::strncpy(buf, s.c_str(), buf_len - 1);
    buf[buf_len - 1] = 0;
  }
  return (int)DialectOps(base_op).size();
}
}
