// Registry behaviour of the RAF-style shim, after tests/cpp/test_op_dialect.cc:72-102 of the reference:
// two fake dialects register the same base op with different priorities; dispatch tries the higher
// priority first and falls through when its maker declines.
#include <cstdio>
#include <string>

#include "raf_shim.h"

using namespace raf_shim;

struct FakeEnv : OpEnv {
  std::string n;
  explicit FakeEnv(std::string name) : n(std::move(name)) {}
  std::string name() const override { return n; }
  void Execute(const CallValues&) override {}
  void Execute(const std::vector<Value>&, Value) override {}
};

static bool decline_high = false;
static OpEnv* MakeHigh(const CallValues&) { return decline_high ? nullptr : new FakeEnv("raf.op.fake_hi.probe"); }
static OpEnv* MakeLow(const CallValues&) { return new FakeEnv("raf.op.fake_lo.probe"); }

RAF_REGISTER_DIALECT_OP(fake_lo, probe, 5);
RAF_OP_ENV_MAKER("raf.op.fake_lo.probe", MakeLow);
RAF_REGISTER_DIALECT_OP(fake_hi, probe, 30);
RAF_OP_ENV_MAKER("raf.op.fake_hi.probe", MakeHigh);

#define EXPECT(c)                                         \
  do {                                                    \
    if (!(c)) {                                           \
      std::printf("FAILED %s:%d %s\n", __FILE__, __LINE__, #c); \
      return 1;                                           \
    }                                                     \
  } while (0)

int main() {
  auto ops = DialectOps("raf.op.probe");
  EXPECT(ops.size() == 2);
  EXPECT(ops[0].dialect == "fake_hi" && ops[0].plevel == 30);
  EXPECT(ops[1].dialect == "fake_lo" && ops[1].plevel == 5);
  CallValues cv;
  cv.op = "raf.op.probe";
  EXPECT(Dispatch(cv)->name() == "raf.op.fake_hi.probe");
  decline_high = true;
  EXPECT(Dispatch(cv)->name() == "raf.op.fake_lo.probe");
  cv.op = "raf.op.no_such_op";
  bool threw = false;
  try {
    Dispatch(cv);
  } catch (const Error&) {
    threw = true;
  }
  EXPECT(threw);
  // requests are recorded for the executor
  FakeEnv env("x");
  void* ws = nullptr;
  void* st = nullptr;
  env.RequestWorkspace(&ws, Device(), 128);
  env.RequestStream(&st, Device(), kCudaCommunicate);
  EXPECT(env.GetRequests().workspace.size() == 1 && env.GetRequests().workspace[0].nbytes == 128);
  EXPECT(env.GetRequests().stream.size() == 1 && env.GetRequests().stream[0].tag_idx == 4);
  std::printf("raf shim ok\n");
  return 0;
}
