// A minimal restatement of RAF's operator boundary, enough to host the MoE hot-path operators
// the way the reference hosts them: an OpEnv per (op, shapes), created by a maker registered
// under the dialect-qualified name, found through a priority-ordered dialect list.
//
// Mirrors (paths inside the reference project): include/raf/op.h:55-91 (OpEnv, requests),
// :329-332 (RAF_OP_ENV_MAKER), include/raf/dialect.h:234-242 (RAF_REGISTER_DIALECT_OP),
// src/impl/op.cc:130-199 (Dispatch: walk the dialects by priority until a maker accepts),
// src/requests.h:17-52 (workspace / stream / distributed requests filled in by the executor).
// TVM's object system is replaced by plain structs; nothing else is modelled.
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace raf_shim {

struct Device {
  int device_type = 2;  // 1 = cpu, 2 = cuda
  int device_id = 0;
};

enum DTypeCode { kInt = 0, kUInt = 1, kFloat = 2, kBFloat = 4 };
struct DType {
  int code = kFloat;
  int bits = 32;
  bool operator==(const DType& o) const { return code == o.code && bits == o.bits; }
};

// Stand-in for DLTensor: a view of executor-owned memory.
struct Tensor {
  void* data = nullptr;
  Device device;
  DType dtype;
  std::vector<int64_t> shape;
  int64_t numel() const {
    int64_t n = 1;
    for (int64_t s : shape) n *= s;
    return n;
  }
  int64_t nbytes() const { return numel() * (dtype.bits / 8); }
};

struct Value {
  enum Kind { kNone, kTensor, kTuple, kInt, kFloat } kind = kNone;
  Tensor tensor;
  std::vector<Value> fields;
  int64_t i = 0;
  double f = 0;
  static Value T(const Tensor& t) { Value v; v.kind = kTensor; v.tensor = t; return v; }
  static Value Tuple(std::vector<Value> f) { Value v; v.kind = kTuple; v.fields = std::move(f); return v; }
  static Value Int(int64_t x) { Value v; v.kind = kInt; v.i = x; v.f = (double)x; return v; }
  static Value Float(double x) { Value v; v.kind = kFloat; v.f = x; v.i = (int64_t)x; return v; }
};

// One call: arguments in schema order (scripts/src_codegen/def_schema.py of the reference), the
// pre-allocated output and the device.
struct CallValues {
  std::string op;  // base name, e.g. "raf.op.moe_encode"
  std::vector<Value> args;
  Value out;
  Device device;
};

struct Requests {
  struct Workspace { void** dest; Device device; int64_t nbytes; };
  struct Stream { void** dest; Device device; int tag_idx; };
  struct Distributed { void** dest; };
  std::vector<Workspace> workspace;
  std::vector<Stream> stream;
  std::vector<Distributed> distributed;
};

enum StreamTag { kCudaCompute = 1, kMemCpuToCuda = 2, kMemCudaToCpu = 3, kCudaCommunicate = 4 };

struct Error : std::runtime_error {
  using std::runtime_error::runtime_error;
};
#define RAF_SHIM_CHECK(cond, msg)                                   \
  do {                                                              \
    if (!(cond)) throw ::raf_shim::Error(std::string("Check failed: " #cond ": ") + (msg)); \
  } while (0)

class OpEnv {
 public:
  virtual ~OpEnv() = default;
  virtual std::string name() const = 0;
  virtual void Execute(const CallValues& call) = 0;
  virtual void Execute(const std::vector<Value>& inputs, Value output) = 0;
  void RequestWorkspace(void** dest, const Device& device, int64_t nbytes) { requests_.workspace.push_back({dest, device, nbytes}); }
  void RequestStream(void** dest, const Device& device, int tag_idx) { requests_.stream.push_back({dest, device, tag_idx}); }
  void RequestDistributed(void** dest) { requests_.distributed.push_back({dest}); }
  const Requests& GetRequests() const { return requests_; }
  std::vector<int> arg_indices;

 private:
  Requests requests_;
};

using FMakeOpEnv = std::function<OpEnv*(const CallValues&)>;
using FDeclare = std::function<void(CallValues*)>;

struct DialectEntry {
  std::string dialect, dialect_op;
  int plevel;
};

// Registries (process-global, filled by static initialisers like the reference's).
bool RegisterOpEnvMaker(const std::string& dialect_op, FMakeOpEnv maker);
bool RegisterDialectOp(const std::string& dialect, const std::string& base_op, const std::string& dialect_op, int plevel);
bool RegisterDeclare(const std::string& base_op, FDeclare fn);
std::vector<DialectEntry> DialectOps(const std::string& base_op);  // sorted by descending plevel
std::vector<std::string> RegisteredOps();

// Output shapes and dtypes of a call (fills call->out with tensors whose data is null).
void Declare(CallValues* call);
// The first dialect op, by priority, whose maker accepts the call.  Throws if none does.
std::shared_ptr<OpEnv> Dispatch(const CallValues& call);

// The stream cuda-dialect operators launch on (DeviceAPI::GetStream of the reference,
// src/device_api/cuda/cuda.cc:194-203), and the communicator handed out by RequestDistributed.
void SetStream(void* stream);
void* GetStream();
void SetCommunicator(void* comm, int rank, int size);
void* GetCommunicator();
int GetCommunicatorSize();  // DistContext::Global()->size of the reference

#define RAF_SHIM_CONCAT_(a, b) a##b
#define RAF_SHIM_CONCAT(a, b) RAF_SHIM_CONCAT_(a, b)
#define RAF_OP_ENV_MAKER(DIALECT_OP_NAME, MAKER) \
  static bool RAF_SHIM_CONCAT(_raf_op_env_maker_, __COUNTER__) = ::raf_shim::RegisterOpEnvMaker(DIALECT_OP_NAME, MAKER)
#define RAF_REGISTER_DIALECT_OP(DIALECT, OP, PLEVEL)                  \
  static bool RAF_SHIM_CONCAT(_raf_dialect_op_, __COUNTER__) =        \
      ::raf_shim::RegisterDialectOp(#DIALECT, "raf.op." #OP, "raf.op." #DIALECT "." #OP, PLEVEL)
#define RAF_OP_DECLARE(OP_NAME, BODY) \
  static bool RAF_SHIM_CONCAT(_raf_op_declare_, __COUNTER__) = ::raf_shim::RegisterDeclare(OP_NAME, BODY)

}  // namespace raf_shim
