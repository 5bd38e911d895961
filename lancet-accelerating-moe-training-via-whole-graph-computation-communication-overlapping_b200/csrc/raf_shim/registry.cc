#include <algorithm>
#include <map>
#include <mutex>

#include "raf_shim.h"

namespace raf_shim {
namespace {
struct Registry {
  std::map<std::string, FMakeOpEnv> makers;
  std::map<std::string, std::vector<DialectEntry>> dialects;
  std::map<std::string, FDeclare> declares;
  void* stream = nullptr;
  void* comm = nullptr;
  int rank = 0, size = 1;
};
Registry& R() {
  static Registry r;
  return r;
}
}  // namespace

bool RegisterOpEnvMaker(const std::string& dialect_op, FMakeOpEnv maker) {
  R().makers[dialect_op] = std::move(maker);
  return true;
}

bool RegisterDialectOp(const std::string& dialect, const std::string& base_op, const std::string& dialect_op, int plevel) {
  auto& v = R().dialects[base_op];
  for (auto& e : v)
    if (e.dialect == dialect) {
      e = {dialect, dialect_op, plevel};
      std::stable_sort(v.begin(), v.end(), [](const DialectEntry& a, const DialectEntry& b) { return a.plevel > b.plevel; });
      return true;
    }
  v.push_back({dialect, dialect_op, plevel});
  std::stable_sort(v.begin(), v.end(), [](const DialectEntry& a, const DialectEntry& b) { return a.plevel > b.plevel; });
  return true;
}

bool RegisterDeclare(const std::string& base_op, FDeclare fn) {
  R().declares[base_op] = std::move(fn);
  return true;
}

std::vector<DialectEntry> DialectOps(const std::string& base_op) {
  auto it = R().dialects.find(base_op);
  return it == R().dialects.end() ? std::vector<DialectEntry>() : it->second;
}

std::vector<std::string> RegisteredOps() {
  std::vector<std::string> out;
  for (auto& kv : R().makers) out.push_back(kv.first);
  return out;
}

void Declare(CallValues* call) {
  auto it = R().declares.find(call->op);
  if (it == R().declares.end()) throw Error("no declaration registered for " + call->op);
  it->second(call);
}

std::shared_ptr<OpEnv> Dispatch(const CallValues& call) {
  std::string errors;
  for (const DialectEntry& e : DialectOps(call.op)) {
    auto mk = R().makers.find(e.dialect_op);
    if (mk == R().makers.end()) continue;
    OpEnv* env = nullptr;
    try {
      env = mk->second(call);
    } catch (const Error& err) {
      errors += "\n  " + e.dialect_op + ": " + err.what();
      continue;
    }
    if (env) return std::shared_ptr<OpEnv>(env);
    errors += "\n  " + e.dialect_op + ": declined";
  }
  throw Error("Cannot dispatch " + call.op + ": no dialect op accepted the call" + errors);
}

void SetStream(void* stream) { R().stream = stream; }
void* GetStream() { return R().stream; }
void SetCommunicator(void* comm, int rank, int size) {
  R().comm = comm;
  R().rank = rank;
  R().size = size;
}
void* GetCommunicator() { return R().comm; }
int GetCommunicatorSize() { return R().size; }

}  // namespace raf_shim
