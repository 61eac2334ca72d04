// The kuiper-style layer API of this repository against the CPU oracle, in the idiom of the
// reference's op tests (CUDA kernel vs CPU kernel, exact for copies, NEAR for attention;
// compare test/test_op/test_cu_rmsnorm.cpp:8-38 in the reference).  Test infrastructure:
// links the oracle; the product headers never do.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "base/paged_kv.h"
#include "model/kv_cache_view.h"
#include "op/batched_rope.h"
#include "op/flash_attention.h"
#include "op/kv_cache.h"
#include "op/mha.h"
#include "op/misc_layers.h"
#include "op/rope.h"

extern "C" {
void orc_sin_cos_cache(int32_t, int32_t, float, float*, float*);
void orc_rope(int32_t, int32_t, int32_t, float*, float*, int32_t, const float*, const float*);
void orc_rope_batched(int32_t, int32_t, int32_t, int32_t, int32_t, float*, float*, const float*, const float*);
void orc_mha(int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, float*, const float*, float*,
             const float*, const float*);
void orc_mha_prefill(int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, int32_t, float*, const float*,
                     const float*, const float*, int32_t);
}

static int g_fail = 0, g_checks = 0;
#define EXPECT(cond)                                                          \
  do {                                                                        \
    ++g_checks;                                                               \
    if (!(cond)) {                                                            \
      ++g_fail;                                                               \
      std::printf("  FAILED %s (%s:%d)\n", #cond, __FILE__, __LINE__);        \
    }                                                                         \
  } while (0)

static float max_abs_diff(const std::vector<float>& a, const std::vector<float>& b) {
  float m = 0.f;
  for (size_t i = 0; i < a.size(); ++i) {
    float d = std::fabs(a[i] - b[i]);
    if (!(d <= m)) m = std::isnan(d) ? INFINITY : d;
  }
  return m;
}

using base::DataType;
using base::DeviceType;
static auto cuda_alloc() { return base::CUDADeviceAllocatorFactory::get_instance(); }

template <typename T>
static tensor::Tensor device_tensor(DataType dt, std::vector<int32_t> dims, const std::vector<T>& host) {
  tensor::Tensor t(dt, dims, true, cuda_alloc());
  cudaMemcpy(t.ptr<void>(), host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice);
  return t;
}
template <typename T>
static std::vector<T> to_host(const tensor::Tensor& t) {
  std::vector<T> h(t.byte_size() / sizeof(T));
  cudaMemcpy(h.data(), t.ptr<void>(), t.byte_size(), cudaMemcpyDeviceToHost);
  return h;
}
static std::vector<__half> to_half(const std::vector<float>& v) {
  std::vector<__half> h(v.size());
  for (size_t i = 0; i < v.size(); ++i) h[i] = __float2half_rn(v[i]);
  return h;
}
static std::vector<float> from_half(const std::vector<__half>& v) {
  std::vector<float> f(v.size());
  for (size_t i = 0; i < v.size(); ++i) f[i] = __half2float(v[i]);
  return f;
}
static std::vector<float> randn(size_t n, std::mt19937_64& g) {
  std::normal_distribution<float> d(0.f, 1.f);
  std::vector<float> v(n);
  for (auto& x : v) x = d(g);
  return v;
}

// The CPU-runnable anchor case: Qwen2.5-1.5B attention shape, 512 cached + 1 new token, fp32, RoPE
// theta 1e6 on the new Q/K, contiguous cache, through RoPELayer -> KVCacheLayer -> MHA.
static void test_config1_fp32_layers() {
  std::printf("config 1 through RoPEGpuPosLayer / KVCacheLayer / MultiHeadAttention (fp32)\n");
  const int H = 12, HKV = 2, D = 128, S = 600, L = 2, layer = 1, pos = 512;
  const int dim = H * D, kv_dim = HKV * D;
  std::mt19937_64 g(42);
  std::vector<float> kc = randn(size_t(L) * S * kv_dim, g), vc = randn(size_t(L) * S * kv_dim, g);
  std::vector<float> q = randn(dim, g), k = randn(kv_dim, g), v = randn(kv_dim, g);
  std::vector<float> sin(size_t(S) * D), cos(size_t(S) * D);
  orc_sin_cos_cache(D, S, 1e6f, sin.data(), cos.data());
  // oracle
  std::vector<float> q_ref = q, k_ref = k, kc_ref = kc, vc_ref = vc, score(size_t(H) * S), out_ref(dim);
  orc_rope(dim, kv_dim, D, q_ref.data(), k_ref.data(), pos, sin.data(), cos.data());
  std::memcpy(&kc_ref[(size_t(layer) * S + pos) * kv_dim], k_ref.data(), kv_dim * 4);
  std::memcpy(&vc_ref[(size_t(layer) * S + pos) * kv_dim], v.data(), kv_dim * 4);
  orc_mha(pos, H, layer, S, kv_dim, H / HKV, D, out_ref.data(), q_ref.data(), score.data(), kc_ref.data(), vc_ref.data());
  // device, reference call order: rope -> store K, V -> attend
  auto cfg = std::make_shared<kernel::CudaConfig>();
  cfg->init();
  tensor::Tensor dq = device_tensor(DataType::kDataTypeFp32, {dim}, q), dk = device_tensor(DataType::kDataTypeFp32, {kv_dim}, k);
  tensor::Tensor dv = device_tensor(DataType::kDataTypeFp32, {kv_dim}, v);
  tensor::Tensor dkc = device_tensor(DataType::kDataTypeFp32, {L, S, kv_dim}, kc), dvc = device_tensor(DataType::kDataTypeFp32, {L, S, kv_dim}, vc);
  tensor::Tensor dsin = device_tensor(DataType::kDataTypeFp32, {S, D}, sin), dcos = device_tensor(DataType::kDataTypeFp32, {S, D}, cos);
  tensor::Tensor dpos = device_tensor(DataType::kDataTypeInt32, {1}, std::vector<int32_t>{pos});
  tensor::Tensor dout(DataType::kDataTypeFp32, dim, true, cuda_alloc());
  tensor::Tensor dscore(DataType::kDataTypeFp32, H, S, true, cuda_alloc());
  op::RoPEGpuPosLayer rope(DeviceType::kDeviceCUDA, dim, kv_dim, D);
  rope.set_cuda_config(cfg);
  rope.set_input(0, dq); rope.set_input(1, dk); rope.set_input(2, dpos); rope.set_input(3, dsin); rope.set_input(4, dcos);
  EXPECT(bool(rope.forward()));
  op::KVCacheLayer kstore(DeviceType::kDeviceCUDA, kv_dim, S), vstore(DeviceType::kDeviceCUDA, kv_dim, S);
  for (op::KVCacheLayer* st : {&kstore, &vstore}) { st->set_cuda_config(cfg); st->set_layer_index(layer); st->set_use_gpu_pos(true); }
  kstore.set_input(0, dk); kstore.set_input(1, dkc); kstore.set_input(2, dpos);
  vstore.set_input(0, dv); vstore.set_input(1, dvc); vstore.set_input(2, dpos);
  EXPECT(bool(kstore.forward()));
  EXPECT(bool(vstore.forward()));
  op::MultiHeadAttention mha(DeviceType::kDeviceCUDA, layer, H / HKV, kv_dim, S, H, D);
  mha.set_cuda_config(cfg);
  mha.set_pos(pos);
  mha.set_input(0, dq); mha.set_input(1, dscore); mha.set_input(2, dkc); mha.set_input(3, dvc);
  mha.set_output(0, dout);
  EXPECT(bool(mha.forward()));
  cudaStreamSynchronize(cfg->stream);
  EXPECT(to_host<float>(dq) == q_ref);    // RoPE'd q bit-exact
  EXPECT(to_host<float>(dkc) == kc_ref);  // appended cache contents bit-exact
  EXPECT(to_host<float>(dvc) == vc_ref);
  float err = max_abs_diff(to_host<float>(dout), out_ref);
  std::printf("  attention max abs err %.3e\n", err);
  EXPECT(err < 1e-5f);
  // same through the device-position layer
  op::MHAGpuPosLayer gp(DeviceType::kDeviceCUDA);
  gp.set_cuda_config(cfg);
  tensor::Tensor dout2(DataType::kDataTypeFp32, dim, true, cuda_alloc());
  EXPECT(bool(gp.forward(dpos.ptr<int32_t>(), H, layer, S, kv_dim, H / HKV, D, dout2, dq, dscore, dkc, dvc)));
  cudaStreamSynchronize(cfg->stream);
  EXPECT(max_abs_diff(to_host<float>(dout2), out_ref) < 1e-5f);
  // the eager path's "slot mapping": views aliasing cache[layer][pos] (Model::slice_kv_cache)
  auto views = model::slice_kv_cache(dkc, dvc, layer, pos, S, kv_dim);
  EXPECT(views.first.size() == size_t(kv_dim) && views.second.size() == size_t(kv_dim));
  EXPECT(views.first.ptr<float>() == dkc.ptr<float>() + (size_t(layer) * S + pos) * kv_dim);
  EXPECT(views.first.device_type() == DeviceType::kDeviceCUDA);
  EXPECT(to_host<float>(views.first) == k_ref);   // the row the store layer wrote
  EXPECT(to_host<float>(views.second) == v);
  const int32_t row[3] = {7, 2, -1};
  EXPECT(model::paged_slot(row, 3, 16, 0) == 7 * 16 && model::paged_slot(row, 3, 16, 17) == 2 * 16 + 1);
  EXPECT(model::paged_slot(row, 3, 16, 40) == -1 && model::paged_slot(row, 3, 16, 48) == -1);
}

// fp16 decode through FlashAttentionDecodeLayer (host pos and device pos) + CopyToKVCacheLayer.
static void test_flash_decode_fp16() {
  std::printf("FlashAttentionDecodeLayer fp16 (Qwen3-8B shape), host and device position\n");
  const int H = 32, HKV = 8, D = 128, S = 400, L = 1, pos = 290;
  const int dim = H * D, kv_dim = HKV * D;
  std::mt19937_64 g(7);
  std::vector<__half> kc = to_half(randn(size_t(L) * S * kv_dim, g)), vc = to_half(randn(size_t(L) * S * kv_dim, g));
  std::vector<__half> q = to_half(randn(dim, g)), knew = to_half(randn(kv_dim, g));
  std::vector<__half> kc_ref = kc;
  std::memcpy(&kc_ref[size_t(pos) * kv_dim], knew.data(), kv_dim * 2);
  std::vector<float> score(size_t(H) * S), out_ref(dim);
  std::vector<float> qf = from_half(q), kf = from_half(kc_ref), vf = from_half(vc);
  orc_mha(pos, H, 0, S, kv_dim, H / HKV, D, out_ref.data(), qf.data(), score.data(), kf.data(), vf.data());
  auto cfg = std::make_shared<kernel::CudaConfig>();
  cfg->init();
  tensor::Tensor dq = device_tensor(DataType::kDataTypeFp16, {dim}, q), dkn = device_tensor(DataType::kDataTypeFp16, {kv_dim}, knew);
  tensor::Tensor dkc = device_tensor(DataType::kDataTypeFp16, {L, S, kv_dim}, kc), dvc = device_tensor(DataType::kDataTypeFp16, {L, S, kv_dim}, vc);
  tensor::Tensor dpos = device_tensor(DataType::kDataTypeInt32, {1}, std::vector<int32_t>{pos});
  op::CopyToKVCacheLayer cp(DeviceType::kDeviceCUDA);
  cp.set_cuda_config(cfg);
  EXPECT(bool(cp.forward(dkc, dkn, dpos.ptr<int32_t>(), kv_dim, 0, S)));
  for (int gpu_pos = 0; gpu_pos < 2; ++gpu_pos) {
    tensor::Tensor dout(DataType::kDataTypeFp16, dim, true, cuda_alloc());
    op::FlashAttentionDecodeLayer fa(DeviceType::kDeviceCUDA, H, HKV, D, H / HKV, S, kv_dim, true);
    fa.set_cuda_config(cfg);
    fa.set_attention_type(gpu_pos ? base::AttentionType::kAttentionFlash2 : base::AttentionType::kAttentionFlash1);
    fa.set_layer_index(0);
    fa.set_pos(pos);
    fa.set_use_gpu_pos(gpu_pos != 0);
    fa.set_input(0, dq); fa.set_input(1, dout); fa.set_input(2, dkc); fa.set_input(3, dvc); fa.set_input(4, dpos);
    EXPECT(bool(fa.forward()));
    cudaStreamSynchronize(cfg->stream);
    float err = max_abs_diff(from_half(to_host<__half>(dout)), out_ref);
    std::printf("  gpu_pos=%d max abs err %.3e\n", gpu_pos, err);
    EXPECT(err <= 2e-3f);
  }
  EXPECT(std::memcmp(to_host<__half>(dkc).data(), kc_ref.data(), kc_ref.size() * 2) == 0);
}

// Prefill chunk with start_pos > 0: BatchedRoPELayer -> FusedKVCacheUpdateLayer ->
// FlashAttentionPrefillLayer / BatchedMHALayer, fp32 contiguous cache.
static void test_prefill_chunk_fp32() {
  std::printf("prefill chunk (start_pos 40, 24 tokens) through the batched layers (fp32)\n");
  const int H = 8, HKV = 2, D = 128, S = 96, start = 40, n = 24;
  const int dim = H * D, kv_dim = HKV * D;
  std::mt19937_64 g(3);
  std::vector<float> kc = randn(size_t(S) * kv_dim, g), vc = randn(size_t(S) * kv_dim, g);
  std::vector<float> q = randn(size_t(n) * dim, g), k = randn(size_t(n) * kv_dim, g), v = randn(size_t(n) * kv_dim, g);
  std::vector<float> sin(size_t(S) * D), cos(size_t(S) * D);
  orc_sin_cos_cache(D, S, 1e6f, sin.data(), cos.data());
  std::vector<float> q_ref = q, k_ref = k, kc_ref = kc, vc_ref = vc, out_ref(size_t(n) * dim);
  orc_rope_batched(start, n, dim, kv_dim, D, q_ref.data(), k_ref.data(), sin.data(), cos.data());
  std::memcpy(&kc_ref[size_t(start) * kv_dim], k_ref.data(), k_ref.size() * 4);
  std::memcpy(&vc_ref[size_t(start) * kv_dim], v.data(), v.size() * 4);
  orc_mha_prefill(start, n, H, 0, S, kv_dim, H / HKV, D, out_ref.data(), q_ref.data(), kc_ref.data(), vc_ref.data(), 1);
  auto cfg = std::make_shared<kernel::CudaConfig>();
  cfg->init();
  tensor::Tensor dq = device_tensor(DataType::kDataTypeFp32, {n, dim}, q), dk = device_tensor(DataType::kDataTypeFp32, {n, kv_dim}, k);
  tensor::Tensor dv = device_tensor(DataType::kDataTypeFp32, {n, kv_dim}, v);
  tensor::Tensor dkc = device_tensor(DataType::kDataTypeFp32, {1, S, kv_dim}, kc), dvc = device_tensor(DataType::kDataTypeFp32, {1, S, kv_dim}, vc);
  tensor::Tensor dsin = device_tensor(DataType::kDataTypeFp32, {S, D}, sin), dcos = device_tensor(DataType::kDataTypeFp32, {S, D}, cos);
  op::BatchedRoPELayer rope(DeviceType::kDeviceCUDA, dim, kv_dim, D, H, HKV);
  rope.set_cuda_config(cfg);
  rope.set_seq_len(n);
  rope.set_start_pos(start);
  rope.set_input(0, dq); rope.set_input(1, dk); rope.set_input(2, dsin); rope.set_input(3, dcos);
  EXPECT(bool(rope.forward()));
  op::FusedKVCacheUpdateLayer upd(DeviceType::kDeviceCUDA);
  upd.set_cuda_config(cfg);
  EXPECT(bool(upd.forward(dk, dv, dkc, dvc, 0, start, n, kv_dim, S)));
  tensor::Tensor dout(DataType::kDataTypeFp32, n, dim, true, cuda_alloc());
  op::FlashAttentionPrefillLayer fa(DeviceType::kDeviceCUDA, H, HKV, D, S);
  fa.set_cuda_config(cfg);
  fa.set_start_pos(start);
  fa.set_cur_seq_len(n);
  fa.set_layer_index(0);
  fa.set_input(0, dq); fa.set_input(1, dout); fa.set_input(2, dkc); fa.set_input(3, dvc);
  EXPECT(bool(fa.forward()));
  cudaStreamSynchronize(cfg->stream);
  EXPECT(to_host<float>(dq) == q_ref);
  EXPECT(to_host<float>(dkc) == kc_ref);
  EXPECT(to_host<float>(dvc) == vc_ref);
  float err = max_abs_diff(to_host<float>(dout), out_ref);
  std::printf("  flash prefill max abs err %.3e\n", err);
  EXPECT(err < 1e-5f);
  op::BatchedMHALayer bm(DeviceType::kDeviceCUDA);
  bm.set_cuda_config(cfg);
  tensor::Tensor dout2(DataType::kDataTypeFp32, n, dim, true, cuda_alloc());
  tensor::Tensor dscore(DataType::kDataTypeFp32, 1, true, cuda_alloc());
  EXPECT(bool(bm.forward(start, n, H, 0, S, dim, kv_dim, H / HKV, D, dout2, dq, dscore, dkc, dvc)));
  cudaStreamSynchronize(cfg->stream);
  EXPECT(max_abs_diff(to_host<float>(dout2), out_ref) < 1e-5f);
  // a layer without a CudaConfig reports an error instead of crashing
  op::FlashAttentionPrefillLayer bare(DeviceType::kDeviceCUDA, H, HKV, D, S);
  bare.set_input(0, dq); bare.set_input(1, dout); bare.set_input(2, dkc); bare.set_input(3, dvc);
  EXPECT(!bool(bare.forward()));
}

// Paged mode: the same layers on a block pool managed by base::PagedKVManager.
static void test_paged_layers_fp16() {
  std::printf("paged mode: KVCacheLayer.set_slot_mapping + FlashAttentionDecodeLayer.set_paged (fp16)\n");
  const int H = 32, HKV = 8, D = 128, BS = 16, B = 3, NB = 40;
  const int dim = H * D, kv_dim = HKV * D;
  const int lens[B] = {37, 5, 130};
  std::mt19937_64 g(11);
  base::PagedKVConfig pc;
  pc.num_blocks = NB;
  pc.seed = 9;
  base::PagedKVManager mgr(pc);
  std::vector<__half> pool_init(size_t(NB) * HKV * BS * D, __float2half_rn(NAN));
  tensor::Tensor kpool = device_tensor(DataType::kDataTypeFp16, {NB, HKV, BS, D}, pool_init);
  tensor::Tensor vpool = device_tensor(DataType::kDataTypeFp16, {NB, HKV, BS, D}, pool_init);
  auto cfg = std::make_shared<kernel::CudaConfig>();
  cfg->init();
  std::vector<std::vector<float>> kh(B), vh(B);
  std::vector<int32_t> table(size_t(B) * 16, -1), seq_lens(B);
  for (int b = 0; b < B; ++b) {
    int s = mgr.add_sequence();
    std::vector<int64_t> slots;
    EXPECT(bool(mgr.append(s, lens[b], &slots)));
    std::vector<__half> k = to_half(randn(size_t(lens[b]) * kv_dim, g)), v = to_half(randn(size_t(lens[b]) * kv_dim, g));
    kh[b] = from_half(k);
    vh[b] = from_half(v);
    tensor::Tensor dslots = device_tensor(DataType::kDataTypeInt64, {lens[b]}, slots);
    tensor::Tensor dk = device_tensor(DataType::kDataTypeFp16, {lens[b], kv_dim}, k), dv = device_tensor(DataType::kDataTypeFp16, {lens[b], kv_dim}, v);
    op::KVCacheLayer ks(DeviceType::kDeviceCUDA, kv_dim, 0, true), vs(DeviceType::kDeviceCUDA, kv_dim, 0, true);
    ks.set_cuda_config(cfg); vs.set_cuda_config(cfg);
    ks.set_slot_mapping(dslots, lens[b], D, NB); vs.set_slot_mapping(dslots, lens[b], D, NB);
    ks.set_input(0, dk); ks.set_input(1, kpool);
    vs.set_input(0, dv); vs.set_input(1, vpool);
    EXPECT(bool(ks.forward()));
    EXPECT(bool(vs.forward()));
    cudaStreamSynchronize(cfg->stream);
    EXPECT(bool(mgr.fill_block_table_row(s, &table[size_t(b) * 16], 16)));
    seq_lens[b] = lens[b];
  }
  std::vector<__half> q = to_half(randn(size_t(B) * dim, g));
  tensor::Tensor dq = device_tensor(DataType::kDataTypeFp16, {B, dim}, q);
  tensor::Tensor dout(DataType::kDataTypeFp16, B, dim, true, cuda_alloc());
  tensor::Tensor dtable = device_tensor(DataType::kDataTypeInt32, {B, 16}, table);
  tensor::Tensor dlens = device_tensor(DataType::kDataTypeInt32, {B}, seq_lens);
  op::FlashAttentionDecodeLayer fa(DeviceType::kDeviceCUDA, H, HKV, D, H / HKV, 0, kv_dim, true);
  fa.set_cuda_config(cfg);
  fa.set_paged(dtable, dlens, B, NB);
  fa.set_input(0, dq); fa.set_input(1, dout); fa.set_input(2, kpool); fa.set_input(3, vpool);
  EXPECT(bool(fa.forward()));
  cudaStreamSynchronize(cfg->stream);
  // the same step with a plan (made once per step, carried by every layer): the same bits
  {
    tensor::Tensor plan(DataType::kDataTypeInt8, int32_t(kpx_decode_plan_bytes()), true, cuda_alloc());
    fa.set_plan(plan);
    EXPECT(bool(op::MultiHeadAttention::plan_decode_step(fa.paged_args(), kpool, H, HKV, D, cfg.get())));
    tensor::Tensor dout2(DataType::kDataTypeFp16, B, dim, true, cuda_alloc());
    fa.set_input(1, dout2);
    EXPECT(bool(fa.forward()));
    cudaStreamSynchronize(cfg->stream);
    std::vector<__half> a1 = to_host<__half>(dout), a2 = to_host<__half>(dout2);
    EXPECT(std::memcmp(a1.data(), a2.data(), a1.size() * sizeof(__half)) == 0);
    std::printf("  with the step's plan: identical output\n");
  }
  std::vector<float> got = from_half(to_host<__half>(dout)), qf = from_half(q);
  for (int b = 0; b < B; ++b) {
    std::vector<float> score(size_t(H) * lens[b]), ref(dim);
    orc_mha(lens[b] - 1, H, 0, lens[b], kv_dim, H / HKV, D, ref.data(), &qf[size_t(b) * dim], score.data(), kh[b].data(), vh[b].data());
    std::vector<float> mine(got.begin() + size_t(b) * dim, got.begin() + size_t(b + 1) * dim);
    float err = max_abs_diff(mine, ref);
    std::printf("  sequence %d (len %d) max abs err %.3e\n", b, lens[b], err);
    EXPECT(err <= 2e-3f);
  }
}

// Plain multi-head attention, 32 KV heads (Llama-2-7B style): beyond what the library's
// built-in scratch serves, so the adapters must fall back to the CudaConfig's workspace; and
// without a CudaConfig the failure must come back as a Status, not as stale output.
static void test_mha_32_kv_heads_falls_back_to_the_config_workspace() {
  std::printf("MultiHeadAttention / FlashAttentionDecodeLayer, 32 Q = 32 KV heads\n");
  const int H = 32, HKV = 32, D = 128, S = 96, pos = 70;
  const int dim = H * D, kv_dim = HKV * D;
  std::mt19937_64 g(21);
  std::vector<float> kc = randn(size_t(S) * kv_dim, g), vc = randn(size_t(S) * kv_dim, g), q = randn(dim, g);
  std::vector<float> score(size_t(H) * S), out_ref(dim);
  orc_mha(pos, H, 0, S, kv_dim, 1, D, out_ref.data(), q.data(), score.data(), kc.data(), vc.data());
  auto cfg = std::make_shared<kernel::CudaConfig>();
  cfg->init();
  tensor::Tensor dq = device_tensor(DataType::kDataTypeFp32, {dim}, q);
  tensor::Tensor dkc = device_tensor(DataType::kDataTypeFp32, {1, S, kv_dim}, kc), dvc = device_tensor(DataType::kDataTypeFp32, {1, S, kv_dim}, vc);
  tensor::Tensor dscore(DataType::kDataTypeFp32, H, S, true, cuda_alloc());
  {
    tensor::Tensor dout(DataType::kDataTypeFp32, dim, true, cuda_alloc());
    op::MultiHeadAttention mha(DeviceType::kDeviceCUDA, 0, 1, kv_dim, S, H, D);
    mha.set_cuda_config(cfg);
    mha.set_pos(pos);
    mha.set_input(0, dq); mha.set_input(1, dscore); mha.set_input(2, dkc); mha.set_input(3, dvc);
    mha.set_output(0, dout);
    EXPECT(bool(mha.forward()));
    cudaStreamSynchronize(cfg->stream);
    EXPECT(cfg->kv_workspace != nullptr);  // the fallback path ran
    float err = max_abs_diff(to_host<float>(dout), out_ref);
    std::printf("  with a CudaConfig: max abs err %.3e\n", err);
    EXPECT(err <= 2e-3f);
  }
  {
    tensor::Tensor dout(DataType::kDataTypeFp32, dim, true, cuda_alloc());
    op::FlashAttentionDecodeLayer fa(DeviceType::kDeviceCUDA, H, HKV, D, 1, S, kv_dim, false);
    fa.set_cuda_config(cfg);
    fa.set_layer_index(0);
    fa.set_pos(pos);
    fa.set_input(0, dq); fa.set_input(1, dout); fa.set_input(2, dkc); fa.set_input(3, dvc);
    EXPECT(bool(fa.forward()));
    cudaStreamSynchronize(cfg->stream);
    EXPECT(max_abs_diff(to_host<float>(dout), out_ref) <= 2e-3f);
  }
  {
    // no CudaConfig: nowhere to keep a workspace; the kernel function reports and changes nothing
    tensor::Tensor dout = device_tensor(DataType::kDataTypeFp32, {dim}, std::vector<float>(dim, -7.f));
    std::printf("  (one '[kuiper-b200] ... static scratch' line is expected here)\n");
    kernel::mha_kernel_cu(pos, H, 0, S, kv_dim, 1, D, dout, dq, dscore, dkc, dvc, DeviceType::kDeviceCUDA, nullptr);
    cudaDeviceSynchronize();
    std::vector<float> untouched = to_host<float>(dout);
    EXPECT(untouched[0] == -7.f && untouched[dim - 1] == -7.f);
  }
  {
    // the status a void kernel function met reaches the layer's caller
    cfg->note_status(KPX_ERR_WORKSPACE_TOO_SMALL);
    tensor::Tensor dout(DataType::kDataTypeFp32, dim, true, cuda_alloc());
    op::MultiHeadAttention mha(DeviceType::kDeviceCUDA, 0, 1, kv_dim, S, H, D);
    mha.set_cuda_config(cfg);
    mha.set_pos(pos);
    mha.set_input(0, dq); mha.set_input(1, dscore); mha.set_input(2, dkc); mha.set_input(3, dvc);
    mha.set_output(0, dout);
    base::Status st = mha.forward();
    EXPECT(!st && st.get_err_code() == KPX_ERR_WORKSPACE_TOO_SMALL);
    EXPECT(bool(mha.forward()));  // taken once, then clean again
  }
}

int main() {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    std::printf("no CUDA device: this test needs one (no CPU fallback exists)\n");
    return 2;
  }
  test_config1_fp32_layers();
  test_flash_decode_fp16();
  test_prefill_chunk_fp32();
  test_paged_layers_fp16();
  test_mha_32_kv_heads_falls_back_to_the_config_workspace();
  std::printf("%d checks, %d failed\n", g_checks, g_fail);
  return g_fail ? 1 : 0;
}
