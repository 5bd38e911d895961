// A C++ host driving the operators through the RAF-style registry, the way RAF's interpreter does
// (src/impl/interpreter.cc:246-337 of the reference): Declare -> allocate outputs -> Dispatch -> satisfy the
// workspace / stream requests -> Execute.  Runs moe_encode and moe_decode on config-1-like shapes and checks
// them against a serial CPU loop (the cumulative count per expert of the reference's gen_location_kernel).
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "raf_shim.h"

using namespace raf_shim;

#define CK(x)                                                                 \
  do {                                                                        \
    cudaError_t e_ = (x);                                                     \
    if (e_ != cudaSuccess) {                                                  \
      std::printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
      return 1;                                                               \
    }                                                                         \
  } while (0)

static Tensor DeviceTensor(std::vector<int64_t> shape, DType dt) {
  Tensor t;
  t.shape = shape;
  t.dtype = dt;
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)std::max<int64_t>(t.nbytes(), 1)) != cudaSuccess) std::exit(2);
  t.data = p;
  return t;
}

// what an executor does around Execute
static int Run(CallValues& cv, cudaStream_t stream, std::string* ran) {
  Declare(&cv);
  std::vector<void*> owned;
  std::function<void(Value&)> alloc = [&](Value& v) {
    if (v.kind == Value::kTuple) for (Value& f : v.fields) alloc(f);
    else if (v.kind == Value::kTensor) { v.tensor = DeviceTensor(v.tensor.shape, v.tensor.dtype); }
  };
  alloc(cv.out);
  SetStream(stream);
  std::shared_ptr<OpEnv> env = Dispatch(cv);
  *ran = env->name();
  for (const auto& w : env->GetRequests().workspace) {
    void* p = nullptr;
    CK(cudaMalloc(&p, (size_t)std::max<int64_t>(w.nbytes, 1)));
    owned.push_back(p);
    *w.dest = p;
  }
  for (const auto& s : env->GetRequests().stream) *s.dest = stream;
  env->Execute(cv);
  CK(cudaStreamSynchronize(stream));
  for (void* p : owned) cudaFree(p);
  return 0;
}

// One cached raf.op.cuda.lans OpEnv executed twice with the executor's workspace scribbled over in between (an
// executor may hand the same address to another op between two calls, src/impl/vm/vm.cc:1260-1266 of the reference):
// the result must equal two calls of fresh OpEnvs on a copy of the state.  The step is a device scalar, as RAF passes it.
static int LansCachedEnv(cudaStream_t stream) {
  const std::vector<int64_t> sizes = {5000, 8192, 3, 70000};
  const int n = (int)sizes.size();
  unsigned rng = 777;
  auto next = [&]() { rng = rng * 1664525u + 1013904223u; return (rng >> 8) * (1.0f / 16777216.0f) - 0.5f; };
  std::vector<Tensor> A, B;   // g, p, m, v lists of both copies
  for (int list = 0; list < 4; ++list)
    for (int i = 0; i < n; ++i) {
      std::vector<float> h((size_t)sizes[i]);
      for (auto& v : h) v = list == 3 ? 1e-6f * (next() + 0.5f) : 0.02f * next();
      for (std::vector<Tensor>* dst : {&A, &B}) {
        Tensor t = DeviceTensor({sizes[i]}, {kFloat, 32});
        CK(cudaMemcpy(t.data, h.data(), h.size() * 4, cudaMemcpyHostToDevice));
        dst->push_back(t);
      }
    }
  Tensor step = DeviceTensor({}, {kFloat, 32});
  auto call_for = [&](const std::vector<Tensor>& tl) {
    CallValues cv;
    cv.op = "raf.op.lans";
    std::vector<Value> fields;
    for (const Tensor& t : tl) fields.push_back(Value::T(t));
    cv.args = {Value::Tuple(fields), Value::T(step), Value::Float(1e-3), Value::Float(0.9), Value::Float(0.999), Value::Float(1e-6),
               Value::Int(1), Value::Float(0.01), Value::Int(1), Value::Int(1), Value::Int(1)};
    Declare(&cv);
    return cv;
  };
  SetStream(stream);
  CallValues cvA = call_for(A), cvB = call_for(B);
  std::shared_ptr<OpEnv> cached = Dispatch(cvA);
  if (cached->name() != "raf.op.cuda.lans") { std::printf("FAILED: lans dispatched to %s\n", cached->name().c_str()); return 1; }
  if (cached->GetRequests().workspace.size() != 1) { std::printf("FAILED: lans should request one workspace\n"); return 1; }
  const size_t ws_bytes = (size_t)cached->GetRequests().workspace[0].nbytes;
  void* ws = nullptr;
  CK(cudaMalloc(&ws, ws_bytes));
  for (int it = 1; it <= 2; ++it) {
    const float fstep = (float)it;
    CK(cudaMemcpy(step.data, &fstep, 4, cudaMemcpyHostToDevice));
    // cached OpEnv, same workspace address, contents destroyed since the previous call
    CK(cudaMemset(ws, 0xFF, ws_bytes));
    *cached->GetRequests().workspace[0].dest = ws;
    cached->Execute(cvA);
    CK(cudaStreamSynchronize(stream));
    // fresh OpEnv with its own workspace on the second copy
    std::shared_ptr<OpEnv> fresh = Dispatch(cvB);
    void* ws2 = nullptr;
    CK(cudaMalloc(&ws2, ws_bytes));
    *fresh->GetRequests().workspace[0].dest = ws2;
    fresh->Execute(cvB);
    CK(cudaStreamSynchronize(stream));
    CK(cudaFree(ws2));
  }
  for (size_t t = 0; t < A.size(); ++t) {
    std::vector<float> a((size_t)A[t].numel()), b(a.size());
    CK(cudaMemcpy(a.data(), A[t].data, a.size() * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(b.data(), B[t].data, b.size() * 4, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < a.size(); ++i)
      if (!(a[i] == b[i])) { std::printf("FAILED: lans cached env differs at tensor %zu element %zu: %g vs %g\n", t, i, a[i], b[i]); return 1; }
  }
  // the parameters moved, and stayed finite
  std::vector<float> p0((size_t)sizes[0]);
  CK(cudaMemcpy(p0.data(), A[n].data, p0.size() * 4, cudaMemcpyDeviceToHost));
  for (float v : p0) if (!std::isfinite(v)) { std::printf("FAILED: lans produced a non-finite parameter\n"); return 1; }
  CK(cudaFree(ws));
  return 0;
}

int main() {
  const int S = 2048, E = 8, M = 64;
  const int C = (S + E - 1) / E;
  std::vector<float> x((size_t)S * M), gate((size_t)S * E);
  unsigned rng = 12345;
  auto next = [&]() { rng = rng * 1664525u + 1013904223u; return (rng >> 8) * (1.0f / 16777216.0f); };
  for (auto& v : x) v = next() - 0.5f;
  for (auto& v : gate) v = next();
  cudaStream_t stream;
  CK(cudaStreamCreate(&stream));
  Tensor tx = DeviceTensor({S, M}, {kFloat, 32}), tg = DeviceTensor({S, E}, {kFloat, 32}), tu = DeviceTensor({E}, {kInt, 32});
  CK(cudaMemcpy(tx.data, x.data(), x.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemcpy(tg.data, gate.data(), gate.size() * 4, cudaMemcpyHostToDevice));
  CK(cudaMemset(tu.data, 0, E * 4));

  CallValues enc;
  enc.op = "raf.op.moe_encode";
  enc.args = {Value::T(tx), Value::T(tg), Value::T(tu), Value::Float(1.0)};
  std::string ran;
  if (Run(enc, stream, &ran)) return 1;
  if (ran != "raf.op.cuda.moe_encode") { std::printf("FAILED: dispatched to %s\n", ran.c_str()); return 1; }
  std::vector<int> il(2 * S), cap(E);
  std::vector<float> gs(S), disp((size_t)E * C * M);
  CK(cudaMemcpy(gs.data(), enc.out.fields[0].tensor.data, S * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(il.data(), enc.out.fields[1].tensor.data, 2 * S * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(cap.data(), enc.out.fields[2].tensor.data, E * 4, cudaMemcpyDeviceToHost));
  CK(cudaMemcpy(disp.data(), enc.out.fields[4].tensor.data, disp.size() * 4, cudaMemcpyDeviceToHost));
  // serial reference
  std::vector<int> cnt(E, 0);
  std::vector<float> want((size_t)E * C * M, 0.f);
  for (int s = 0; s < S; ++s) {
    int best = 0;
    for (int e = 1; e < E; ++e) if (gate[(size_t)s * E + e] > gate[(size_t)s * E + best]) best = e;
    const int loc = cnt[best]++;
    const int idx = loc < C ? best : -1;
    if (il[s] != idx || il[S + s] != loc || gs[s] != gate[(size_t)s * E + best]) {
      std::printf("FAILED: token %d got (%d,%d) want (%d,%d)\n", s, il[s], il[S + s], idx, loc);
      return 1;
    }
    if (idx >= 0) for (int m = 0; m < M; ++m) want[((size_t)idx * C + loc) * M + m] = x[(size_t)s * M + m];
  }
  for (int e = 0; e < E; ++e) if (cap[e] != std::min(cnt[e], C)) { std::printf("FAILED: capacity of expert %d\n", e); return 1; }
  for (size_t i = 0; i < want.size(); ++i) if (want[i] != disp[i]) { std::printf("FAILED: dispatched[%zu]\n", i); return 1; }

  CallValues dec;
  dec.op = "raf.op.moe_decode";
  dec.args = {enc.out.fields[4], enc.out.fields[0], enc.out.fields[1]};
  if (Run(dec, stream, &ran)) return 1;
  std::vector<float> out((size_t)S * M);
  CK(cudaMemcpy(out.data(), dec.out.tensor.data, out.size() * 4, cudaMemcpyDeviceToHost));
  for (int s = 0; s < S; ++s)
    for (int m = 0; m < M; ++m) {
      const float w = il[s] >= 0 ? gs[s] * x[(size_t)s * M + m] : 0.f;
      if (out[(size_t)s * M + m] != w) { std::printf("FAILED: combined[%d,%d]\n", s, m); return 1; }
    }
  if (LansCachedEnv(stream)) return 1;
  std::printf("raf host example ok (%s, %s)\n", "raf.op.cuda.moe_encode", ran.c_str());
  return 0;
}
