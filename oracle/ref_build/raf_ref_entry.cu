/*
 * TEST INFRASTRUCTURE ONLY: C entry points over the reference project's own CUDA launchers.
 *
 * The reference's kernel files src/op/dialect/cuda/kernels/{tutel_moe_dispatch,multi_tensor_lans}.cu are compiled
 * unmodified from where they lie (see build_ref.py) and linked with this file into oracle/_ref/libraf_ref_kernels.so.
 * Their launchers are C++ functions of namespace raf::op::cuda (declared in the reference's kernel_util.cuh, included
 * here from the reference tree); this file only gives them unmangled names and marshals pointer lists the way the
 * reference's operator classes do (src/op/dialect/cuda/moe.cc, src/op/dialect/cuda/lans.cc).  The library is used by
 * tests as a checker for the product's kernels on the same GPU; nothing of the product links or loads it.
 *
 * What the operator classes compute with TVM-compiled functions (argmax, one-hot, masked gate, argsort:
 * moe.cc:133-150, :364-371) is not part of these files; tests prepare those inputs on the host.
 */
#include <cmath>
#include <cstdint>
#include <vector>

#include "kernel_util.cuh"

namespace rc = raf::op::cuda;

namespace {
int done(void* stream) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  return static_cast<int>(e);
}
}  // namespace

extern "C" {

// moe.cc:375-380
int raf_ref_gen_location(int* indices, int* in_capused, int* out_locations, int* out_capused, uint64_t* out_elements,
                         int capacity, int samples, int experts, int model_dim, void* stream) {
  rc::launch_gen_location(indices, in_capused, out_locations, out_capused, out_elements, capacity, samples, experts,
                          model_dim, stream);
  return done(stream);
}

// moe.cc:381-395 (capused != nullptr) and moe.cc:669-684 (capused == nullptr); half: 0 = float, 1 = half
int raf_ref_encode_forward(int half_type, int* indices, int* locations, int* capused, void* x, void* dispatched,
                           int samples, int hidden, int capacity, int experts, void* stream) {
  if (half_type) {
    if (capused) rc::launch_encode_forward(indices, locations, capused, static_cast<half*>(x), static_cast<half*>(dispatched), samples, hidden, capacity, experts, stream);
    else rc::launch_encode_forward(indices, locations, static_cast<half*>(x), static_cast<half*>(dispatched), samples, hidden, capacity, experts, stream);
  } else {
    if (capused) rc::launch_encode_forward(indices, locations, capused, static_cast<float*>(x), static_cast<float*>(dispatched), samples, hidden, capacity, experts, stream);
    else rc::launch_encode_forward(indices, locations, static_cast<float*>(x), static_cast<float*>(dispatched), samples, hidden, capacity, experts, stream);
  }
  return done(stream);
}

// moe.cc:1120-1133
int raf_ref_encode_backward_data(int half_type, int* indices, int* locations, void* dx, void* dy_dispatched, int samples,
                                 int hidden, int capacity, int experts, void* stream) {
  if (half_type) rc::launch_encode_backward_data(indices, locations, static_cast<half*>(dx), static_cast<half*>(dy_dispatched), samples, hidden, capacity, experts, stream);
  else rc::launch_encode_backward_data(indices, locations, static_cast<float*>(dx), static_cast<float*>(dy_dispatched), samples, hidden, capacity, experts, stream);
  return done(stream);
}

// moe.cc:1196-1207
int raf_ref_encode_backward_gate(int half_type, void* dy_gates_s, int* indices, void* grad_gates, int samples,
                                 int experts, void* stream) {
  if (half_type) rc::launch_encode_backward_gate(static_cast<half*>(dy_gates_s), indices, static_cast<half*>(grad_gates), samples, experts, stream);
  else rc::launch_encode_backward_gate(static_cast<float*>(dy_gates_s), indices, static_cast<float*>(grad_gates), samples, experts, stream);
  return done(stream);
}

// moe.cc:1276-1291
int raf_ref_decode_forward(int half_type, void* gates_s, int* indices, int* locations, void* decoded, void* expert_output,
                           int samples, int hidden, int capacity, int experts, void* stream) {
  if (half_type) rc::launch_decode_forward(static_cast<half*>(gates_s), indices, locations, static_cast<half*>(decoded), static_cast<half*>(expert_output), samples, hidden, capacity, experts, stream);
  else rc::launch_decode_forward(static_cast<float*>(gates_s), indices, locations, static_cast<float*>(decoded), static_cast<float*>(expert_output), samples, hidden, capacity, experts, stream);
  return done(stream);
}

// moe.cc:1360-1375
int raf_ref_decode_backward_data(int half_type, void* gates_s, int* indices, int* locations, void* dy, void* grad_expert_output,
                                 int samples, int hidden, int capacity, int experts, void* stream) {
  if (half_type) rc::launch_decode_backward_data(static_cast<half*>(gates_s), indices, locations, static_cast<half*>(dy), static_cast<half*>(grad_expert_output), samples, hidden, capacity, experts, stream);
  else rc::launch_decode_backward_data(static_cast<float*>(gates_s), indices, locations, static_cast<float*>(dy), static_cast<float*>(grad_expert_output), samples, hidden, capacity, experts, stream);
  return done(stream);
}

// moe.cc:1446-1460
int raf_ref_decode_backward_gate(int half_type, void* grad_gates_s, int* indices, int* locations, void* dy, void* expert_output,
                                 int samples, int hidden, int capacity, void* stream) {
  if (half_type) rc::launch_decode_backward_gate(static_cast<half*>(grad_gates_s), indices, locations, static_cast<half*>(dy), static_cast<half*>(expert_output), samples, hidden, capacity, stream);
  else rc::launch_decode_backward_gate(static_cast<float*>(grad_gates_s), indices, locations, static_cast<float*>(dy), static_cast<float*>(expert_output), samples, hidden, capacity, stream);
  return done(stream);
}

// moe.cc:654-662; sorted_indices is what the operator's argsort of the masked gate gives (descending)
int raf_ref_gen_location_bpr(int* indices, int* sorted_indices, int* out_locations, bool* dropping_mask, int* out_capused,
                             uint64_t* out_elements, int capacity, int samples_before_partition, int experts, int model_dim,
                             int n_partitions, int partition_id, void* stream) {
  rc::launch_gen_location_bpr(indices, sorted_indices, out_locations, dropping_mask, out_capused, out_elements, capacity,
                              samples_before_partition, experts, model_dim, n_partitions, partition_id, stream);
  return done(stream);
}

// moe.cc:775-801: the operator copies the partitions' device pointers into a device table, indices first.
// dev_table: 2 * n_partition pointers of device memory.  samples must be a multiple of 1024: the kernel reads
// dev_indices1[S + thid] without a bound (tutel_moe_dispatch.cu:232), so callers never pass another size.
int raf_ref_merge_masks(int* const* indices_ptrs, int* const* locations_ptrs, void** dev_table, int* recon_indices,
                        int* recon_locations, int samples, int experts, int n_partition, void* stream) {
  if (samples % 1024 != 0) return -1;
  std::vector<void*> host(2 * n_partition);
  for (int i = 0; i < n_partition; ++i) {
    host[i] = indices_ptrs[i];
    host[n_partition + i] = locations_ptrs[i];
  }
  cudaMemcpyAsync(dev_table, host.data(), sizeof(void*) * host.size(), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
  rc::launch_merge_masks(reinterpret_cast<int**>(dev_table), reinterpret_cast<int**>(dev_table + n_partition), recon_indices,
                         recon_locations, samples, experts, n_partition, stream);
  return done(stream);
}

// moe.cc:887-920
int raf_ref_redispatch(int half_type, void* const* data_ptrs, int* const* indices_ptrs, void** dev_table, void* redispatched,
                       int samples, int hidden, int capacity, int experts, int n_partition, void* stream) {
  std::vector<void*> host(2 * n_partition);
  for (int i = 0; i < n_partition; ++i) {
    host[i] = data_ptrs[i];
    host[n_partition + i] = indices_ptrs[i];
  }
  cudaMemcpyAsync(dev_table, host.data(), sizeof(void*) * host.size(), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
  if (half_type) rc::launch_redispatch(reinterpret_cast<half**>(dev_table), reinterpret_cast<int**>(dev_table + n_partition), static_cast<half*>(redispatched), samples, hidden, capacity, experts, n_partition, stream);
  else rc::launch_redispatch(reinterpret_cast<float**>(dev_table), reinterpret_cast<int**>(dev_table + n_partition), static_cast<float*>(redispatched), samples, hidden, capacity, experts, n_partition, stream);
  return done(stream);
}

// moe.cc:1015-1050
int raf_ref_redispatch_expert_input(int half_type, void* const* data_ptrs, uint64_t* const* mask_ptrs, void** dev_table,
                                    void* redispatched, int local_expert_id, int local_experts, int capacity, int hidden,
                                    int groups, int n_partition, int recv_cnts_scale, void* stream) {
  std::vector<void*> host(2 * n_partition);
  for (int i = 0; i < n_partition; ++i) {
    host[i] = data_ptrs[i];
    host[n_partition + i] = mask_ptrs[i];
  }
  cudaMemcpyAsync(dev_table, host.data(), sizeof(void*) * host.size(), cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
  if (half_type) rc::launch_redispatch_expert_input(reinterpret_cast<half**>(dev_table), reinterpret_cast<uint64_t**>(dev_table + n_partition), static_cast<half*>(redispatched), local_expert_id, local_experts, capacity, hidden, groups, n_partition, recv_cnts_scale, stream);
  else rc::launch_redispatch_expert_input(reinterpret_cast<float**>(dev_table), reinterpret_cast<uint64_t**>(dev_table + n_partition), static_cast<float*>(redispatched), local_expert_id, local_experts, capacity, hidden, groups, n_partition, recv_cnts_scale, stream);
  return done(stream);
}

/* lans.cc:98-141 for fp32 lists: bias corrections from the step, beta3 from grad_averaging, the list in the order
 * [g..., q..., p..., m..., v...] and one call of multi_tensor_lans_cuda<float> with chunk size 65536 (lans.cc:22).
 * One deliberate difference: tensor i's scratch slice q_i starts at the prefix sum of the sizes before it; lans.cc:126-129
 * uses q + numels[i-1], which makes the slices of three or more tensors overlap.  With one or two tensors both agree.
 * q_scratch: sum(numels) floats; norm_scratch: n * max_chunks + 4 * n floats. */
int raf_ref_lans(float* const* g, float* const* p, float* const* m, float* const* v, const int* numels, int n,
                 float* q_scratch, float* norm_scratch, float lr, float beta1, float beta2, float eps, int bias_correction,
                 float weight_decay, int grad_averaging, int mode, int normalize_grad, float fstep, void* stream) {
  const int chunk = 65536;
  std::vector<int> sizes(numels, numels + n);
  int max_chunks = -1;
  for (int t = 0; t < n; ++t) max_chunks = std::max(max_chunks, (sizes[t] + chunk - 1) / chunk);
  int step = static_cast<int>(fstep);
  float bc1 = 1.0f, bc2 = 1.0f;
  if (bias_correction == 1) {
    bc1 = 1 - std::pow(beta1, step);
    bc2 = 1 - std::pow(beta2, step);
  }
  float beta3 = 1.0f;
  if (grad_averaging == 1) beta3 = 1 - beta1;
  std::vector<float*> tlist;
  for (int i = 0; i < n; ++i) tlist.push_back(g[i]);
  size_t off = 0;
  for (int i = 0; i < n; ++i) {
    tlist.push_back(q_scratch + off);
    off += sizes[i];
  }
  for (int i = 0; i < n; ++i) tlist.push_back(p[i]);
  for (int i = 0; i < n; ++i) tlist.push_back(m[i]);
  for (int i = 0; i < n; ++i) tlist.push_back(v[i]);
  float* per_tensor = norm_scratch;
  float* gn = per_tensor + static_cast<size_t>(n) * max_chunks;
  rc::multi_tensor_lans_cuda<float>(chunk, tlist, lr, beta1, beta2, eps, bias_correction, bc1, bc2, beta3, weight_decay,
                                    grad_averaging, mode, normalize_grad != 0, sizes, stream, per_tensor, gn, gn + n,
                                    gn + 2 * n, gn + 3 * n, max_chunks);
  return done(stream);
}

}  // extern "C"
