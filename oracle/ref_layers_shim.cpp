// C-linkage doorway onto the reference's own layer classes.
//
// TEST INFRASTRUCTURE ONLY.  oracle/build_ref_layers.py compiles this file together with every
// translation unit of the reference (read in place from the reference checkout, never copied) into
// oracle/_ref/libcaif_ref_layers.so.  It is used to capture golden vectors from the executing
// reference (CAIF_DeviceFrozenLinear, CAIF_DeviceLoRAAdapter, CAIF_DeviceMoEFrozenExpert, with
// CAIF_Settings::MatmulMode Accuracy_e for fp32 compute) and to time the reference's device path on
// the same GPU as a comparator.  Nothing under caif_b200/ loads it.
//
// Every buffer argument is HOST memory; tensors go up and come down through the reference's own
// FromHostRaw / CopyToHostRaw.  dtype codes are the reference's CAIF_DataType_e values.
#define USE_CAIF_CUDA 1
#include <cuda_runtime.h>

#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "caif_cuda_stream.h"
#include "caif_data_type.h"
#include "caif_device_frozen_linear_base.h"
#include "caif_device_frozen_linear_factory.h"
#include "caif_device_layer.h"
#include "caif_device_lora_adapter.h"
#include "caif_device_lora_adapter_config.h"
#include "caif_device_moe_frozen_expert.h"
#include "caif_device_moe_frozen_expert_config.h"
#include "caif_device_moe_layer.h"
#include "caif_device_moe_layer_factory.h"
#include "caif_moe_overflow_strategy.h"
#include "caif_device_tensor.h"
#include "caif_ops.h"
#include "caif_run_context.h"
#include "caif_safetensors_format.h"
#include "caif_weight_mapper.h"
#include "caif_settings.h"

using namespace instance;
typedef CAIF_DataType::CAIF_DataType_e Dtype_e;

namespace
{
thread_local std::string t_error;

CAIF_CudaStream &stream()
{
  static CAIF_CudaStream s;
  return s;
}

struct Box
{
  std::unique_ptr<CAIF_DeviceLayer> layer;
};

template <typename F>
int guarded(F &&f)
{
  try
  {
    f();
    return 0;
  }
  catch (const std::exception &e)
  {
    t_error = e.what();
    return 1;
  }
  catch (...)
  {
    t_error = "unknown exception";
    return 1;
  }
}

template <typename ComputeT>
std::unique_ptr<CAIF_DeviceLayer> make_lora(Dtype_e sd, const CAIF_DeviceLoRAAdapterConfig &cfg,
                                            std::unique_ptr<CAIF_DeviceLayer> base, uint32_t seed)
{
  switch (sd)
  {
    case Dtype_e::Float32:
      return std::make_unique<CAIF_DeviceLoRAAdapter<ComputeT, float>>(cfg, std::move(base), stream(), seed);
    case Dtype_e::Float16:
      return std::make_unique<CAIF_DeviceLoRAAdapter<ComputeT, __half>>(cfg, std::move(base), stream(), seed);
    case Dtype_e::BFloat16:
      return std::make_unique<CAIF_DeviceLoRAAdapter<ComputeT, __nv_bfloat16>>(cfg, std::move(base), stream(), seed);
    default:
      break;
  }
  throw std::runtime_error("lora: storage dtype must be fp32, fp16 or bf16");
}

std::unique_ptr<CAIF_DeviceFrozenLinearBase> take_frozen(void *handle)
{
  if (handle == nullptr)
  {
    return nullptr;
  }
  Box *box = static_cast<Box *>(handle);
  auto *f = dynamic_cast<CAIF_DeviceFrozenLinearBase *>(box->layer.get());
  if (f == nullptr)
  {
    throw std::runtime_error("handle is not a frozen linear");
  }
  box->layer.release();
  delete box;
  return std::unique_ptr<CAIF_DeviceFrozenLinearBase>(f);
}

template <typename ComputeT, typename StorageT>
std::unique_ptr<CAIF_DeviceLayer> make_expert_cell(const CAIF_DeviceMoEFrozenExpertConfig &cfg, void *gate, void *up,
                                                   void *down)
{
  typename CAIF_DeviceMoEFrozenExpert<ComputeT, StorageT>::FrozenSubLayers_t sub;
  sub.gate = take_frozen(gate);
  sub.up = take_frozen(up);
  sub.down = take_frozen(down);
  return std::make_unique<CAIF_DeviceMoEFrozenExpert<ComputeT, StorageT>>(cfg, std::move(sub), stream());
}

template <typename ComputeT>
std::unique_ptr<CAIF_DeviceLayer> make_expert(Dtype_e sd, const CAIF_DeviceMoEFrozenExpertConfig &cfg, void *gate,
                                              void *up, void *down)
{
  switch (sd)
  {
    case Dtype_e::Float32:
      return make_expert_cell<ComputeT, float>(cfg, gate, up, down);
    case Dtype_e::Float16:
      return make_expert_cell<ComputeT, __half>(cfg, gate, up, down);
    case Dtype_e::BFloat16:
      return make_expert_cell<ComputeT, __nv_bfloat16>(cfg, gate, up, down);
    default:
      break;
  }
  throw std::runtime_error("expert: storage dtype must be fp32, fp16 or bf16");
}

int run(void *handle, bool backward, const void *x, int x_dtype, uint32_t rows, uint32_t last_dim, int training,
        void *out, size_t out_cap, int *out_dtype, size_t *out_bytes)
{
  return guarded([&] {
    Box *box = static_cast<Box *>(handle);
    CAIF_DeviceTensor in = CAIF_DeviceTensor::FromHostRaw(x, {rows, last_dim}, stream(), static_cast<Dtype_e>(x_dtype));
    CAIF_RunContext ctx;
    ctx.SetStream(stream());
    ctx.SetTraining(training != 0);
    ctx.SetPass(backward ? CAIF_RunContext::Pass_e::Backward_e : CAIF_RunContext::Pass_e::Forward_e);
    CAIF_DeviceTensor res = backward ? box->layer->Backward(in, ctx) : box->layer->Forward(in, ctx);
    stream().Synchronize();
    *out_dtype = static_cast<int>(res.Dtype());
    *out_bytes = res.SizeBytes();
    if (res.SizeBytes() > out_cap)
    {
      throw std::runtime_error("result larger than the caller's buffer");
    }
    res.CopyToHostRaw(out);
    stream().Synchronize();
  });
}
}  // namespace

// ---- the reference's whole MoE layer over frozen experts ------------------------------------------
// CAIF_DeviceMoELayer built from expert handles (consumed) with the constructor that takes ready experts
// (include/caif/caif_device_moe_layer.h:101-116): no shared experts, no router noise, no token dropping.
// The router's weight [input_dim, num_experts] (and bias, when used) is overwritten with the caller's raw
// bytes in the storage dtype.  refl_forward / refl_backward / refl_gradient then drive it like any layer.
template <typename ComputeT, typename StorageT>
static std::unique_ptr<CAIF_DeviceLayer> make_moe_layer(void *const *experts, uint32_t num_experts, uint32_t input_dim,
                                                        uint32_t hidden_dim, uint32_t top_k, const void *router_w,
                                                        const void *router_b, int gating_kind, int norm_topk,
                                                        float scaling, float balance_w, float z_w)
{
  typedef CAIF_DeviceMoEExpertBase<ComputeT, StorageT> Expert_t;
  std::vector<std::unique_ptr<Expert_t>> routed;
  for (uint32_t e = 0; e < num_experts; ++e)
  {
    Box *box = static_cast<Box *>(experts[e]);
    Expert_t *typed = dynamic_cast<Expert_t *>(box->layer.get());
    if (typed == nullptr)
    {
      throw std::runtime_error("moe layer: expert handle has another compute / storage type");
    }
    box->layer.release();
    delete box;
    routed.emplace_back(typed);
  }
  std::vector<std::unique_ptr<Expert_t>> shared;
  auto layer = std::make_unique<CAIF_DeviceMoELayer<ComputeT, StorageT>>(
      input_dim, hidden_dim, top_k, router_b != nullptr, 0.0f, 0.0f,
      CAIF_MoEOverflowStrategy::CAIF_MoEOverflowStrategy_e::NoDrop, balance_w, z_w, std::move(routed),
      std::move(shared), stream(), static_cast<CAIF_DeviceMoELayerFactory::GatingKind_e>(gating_kind),
      norm_topk != 0, scaling);
  CAIF_DeviceTensor &w = layer->ParameterTensor(0);
  w.CopyFromHostRaw(router_w, w.SizeBytes());
  if (router_b != nullptr)
  {
    CAIF_DeviceTensor &b = layer->ParameterTensor(1);
    b.CopyFromHostRaw(router_b, b.SizeBytes());
  }
  stream().Synchronize();
  layer->ZeroGradients();
  return layer;
}

extern "C" {

__attribute__((visibility("default"))) const char *refl_last_error(void) { return t_error.c_str(); }

// accuracy != 0: CAIF_Settings::MatmulMode_e::Accuracy_e (full fp32 products for fp32 compute)
__attribute__((visibility("default"))) int refl_set_accuracy(int accuracy)
{
  return guarded([&] {
    CAIF_Settings::SetMatmulMode(accuracy ? CAIF_Settings::MatmulMode_e::Accuracy_e
                                          : CAIF_Settings::MatmulMode_e::Performance_e);
  });
}

// A frozen linear from the factory with its codes and scales loaded.  codes_dtype is the dtype of the
// tensor handed to LoadFromTensor (UInt8 for packed int4, Int8, or a float dtype), codes_count its
// element count.
__attribute__((visibility("default"))) int refl_frozen_create(uint32_t in_dim, uint32_t out_dim, int storage, int compute,
                                                              uint32_t group_size, int cache_fp32, int scheme,
                                                              const void *codes, int codes_dtype, uint32_t codes_count,
                                                              const void *scales, size_t scales_bytes, void **handle)
{
  return guarded([&] {
    auto box = std::make_unique<Box>();
    box->layer = CAIF_DeviceFrozenLinearFactory::Create(in_dim, out_dim, static_cast<Dtype_e>(storage), stream(),
                                                        group_size, cache_fp32 != 0, static_cast<Dtype_e>(compute),
                                                        static_cast<CAIF_Ops::QuantScheme_e>(scheme));
    auto *f = dynamic_cast<CAIF_DeviceFrozenLinearBase *>(box->layer.get());
    CAIF_DeviceTensor t = CAIF_DeviceTensor::FromHostRaw(codes, {codes_count}, stream(), static_cast<Dtype_e>(codes_dtype));
    stream().Synchronize();
    f->LoadFromTensor(std::move(t));
    if (scales != nullptr && scales_bytes > 0)
    {
      f->LoadScalesFromHost(scales, scales_bytes);
    }
    *handle = box.release();
  });
}

// Wraps a frozen linear (the handle is consumed) into a LoRA adapter and overwrites A [rank, in] and
// B [out, rank] with the caller's values (raw bytes in the storage dtype).
__attribute__((visibility("default"))) int refl_lora_wrap(void *base, uint32_t rank, float alpha, uint32_t in_dim,
                                                          uint32_t out_dim, int storage, int compute, const void *a,
                                                          const void *b, void **handle)
{
  return guarded([&] {
    Box *inner = static_cast<Box *>(base);
    const CAIF_DeviceLoRAAdapterConfig cfg(rank, alpha, in_dim, out_dim);
    auto box = std::make_unique<Box>();
    const Dtype_e sd = static_cast<Dtype_e>(storage);
    switch (static_cast<Dtype_e>(compute))
    {
      case Dtype_e::Float32:
        box->layer = make_lora<float>(sd, cfg, std::move(inner->layer), 1);
        break;
      case Dtype_e::Float16:
        box->layer = make_lora<__half>(sd, cfg, std::move(inner->layer), 1);
        break;
      case Dtype_e::BFloat16:
        box->layer = make_lora<__nv_bfloat16>(sd, cfg, std::move(inner->layer), 1);
        break;
      default:
        throw std::runtime_error("lora: compute dtype must be fp32, fp16 or bf16");
    }
    delete inner;
    const size_t n = box->layer->ParameterTensorCount();
    CAIF_DeviceTensor &ta = box->layer->ParameterTensor(n - 2);
    CAIF_DeviceTensor &tb = box->layer->ParameterTensor(n - 1);
    ta.CopyFromHostRaw(a, ta.SizeBytes());
    tb.CopyFromHostRaw(b, tb.SizeBytes());
    stream().Synchronize();
    *handle = box.release();
  });
}

// A frozen expert over three frozen linears (their handles are consumed; gate may be null with use_gated 0).
__attribute__((visibility("default"))) int refl_expert_create(void *gate, void *up, void *down, uint32_t input_dim,
                                                              uint32_t hidden_dim, int use_gated, int storage,
                                                              int compute, void **handle)
{
  return guarded([&] {
    const CAIF_DeviceMoEFrozenExpertConfig cfg(input_dim, hidden_dim, use_gated != 0);
    auto box = std::make_unique<Box>();
    const Dtype_e sd = static_cast<Dtype_e>(storage);
    switch (static_cast<Dtype_e>(compute))
    {
      case Dtype_e::Float32:
        box->layer = make_expert<float>(sd, cfg, gate, up, down);
        break;
      case Dtype_e::Float16:
        box->layer = make_expert<__half>(sd, cfg, gate, up, down);
        break;
      case Dtype_e::BFloat16:
        box->layer = make_expert<__nv_bfloat16>(sd, cfg, gate, up, down);
        break;
      default:
        throw std::runtime_error("expert: compute dtype must be fp32, fp16 or bf16");
    }
    *handle = box.release();
  });
}

__attribute__((visibility("default"))) int refl_forward(void *handle, const void *x, int x_dtype, uint32_t rows,
                                                        uint32_t last_dim, int training, void *out, size_t out_cap,
                                                        int *out_dtype, size_t *out_bytes)
{
  return run(handle, false, x, x_dtype, rows, last_dim, training, out, out_cap, out_dtype, out_bytes);
}

__attribute__((visibility("default"))) int refl_backward(void *handle, const void *dy, int dy_dtype, uint32_t rows,
                                                         uint32_t last_dim, void *out, size_t out_cap, int *out_dtype,
                                                         size_t *out_bytes)
{
  return run(handle, true, dy, dy_dtype, rows, last_dim, 1, out, out_cap, out_dtype, out_bytes);
}

// Gradient tensor `index_from_end` counted from the last parameter (1 = last: LoRA B, 2 = LoRA A), raw bytes.
__attribute__((visibility("default"))) int refl_gradient(void *handle, uint32_t index_from_end, void *out, size_t out_cap,
                                                         size_t *out_bytes)
{
  return guarded([&] {
    Box *box = static_cast<Box *>(handle);
    const size_t n = box->layer->ParameterTensorCount();
    const CAIF_DeviceTensor &t = box->layer->GradientTensor(n - index_from_end);
    *out_bytes = t.SizeBytes();
    if (t.SizeBytes() > out_cap)
    {
      throw std::runtime_error("gradient larger than the caller's buffer");
    }
    t.CopyToHostRaw(out);
    stream().Synchronize();
  });
}

// Times `iters` forward (and, with backward != 0, forward + backward) calls of a layer on a
// [rows, last_dim] input that already sits on the device, with CUDA events on the layer's stream.
// The first `warm` calls are not timed (the reference's cuBLAS-Lt wrapper probes algorithms on the
// first call of a shape, and cache_fp32 keeps the dequantized weight after it).
__attribute__((visibility("default"))) int refl_time(void *handle, const void *x, int x_dtype, const void *dy,
                                                     int dy_dtype, uint32_t rows, uint32_t in_dim, uint32_t out_dim,
                                                     int backward, int warm, int iters, float *ms_per_iter)
{
  return guarded([&] {
    Box *box = static_cast<Box *>(handle);
    CAIF_DeviceTensor in = CAIF_DeviceTensor::FromHostRaw(x, {rows, in_dim}, stream(), static_cast<Dtype_e>(x_dtype));
    CAIF_DeviceTensor grad;
    if (backward)
    {
      grad = CAIF_DeviceTensor::FromHostRaw(dy, {rows, out_dim}, stream(), static_cast<Dtype_e>(dy_dtype));
    }
    CAIF_RunContext ctx;
    ctx.SetStream(stream());
    ctx.SetTraining(backward != 0);
    auto once = [&]() {
      ctx.SetPass(CAIF_RunContext::Pass_e::Forward_e);
      CAIF_DeviceTensor y = box->layer->Forward(in, ctx);
      if (backward)
      {
        ctx.SetPass(CAIF_RunContext::Pass_e::Backward_e);
        CAIF_DeviceTensor dx = box->layer->Backward(grad, ctx);
      }
    };
    for (int i = 0; i < warm; ++i)
    {
      once();
    }
    stream().Synchronize();
    cudaEvent_t e0;
    cudaEvent_t e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, stream().Handle());
    for (int i = 0; i < iters; ++i)
    {
      once();
    }
    cudaEventRecord(e1, stream().Handle());
    cudaEventSynchronize(e1);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms_per_iter = ms / static_cast<float>(iters);
  });
}

// ---- the reference's Host_e path: CAIF_Ops::MatMul / MatMulTransposeA / MatMulTransposeB on host tensors
// (src/caif_ops_host.cpp:54-139 -> src/caif_host_gemm.cpp -> cblas_sgemm).  No GPU is touched.

// An fp32 [rows, cols] tensor in the reference's host memory; *data points at its storage.
__attribute__((visibility("default"))) int refl_host_tensor(uint32_t rows, uint32_t cols, void **handle, float **data)
{
  return guarded([&] {
    auto *t = new CAIF_DeviceTensor(CAIF_DeviceTensor::UninitializedHost({rows, cols}));
    *handle = t;
    *data = static_cast<float *>(t->DeviceDataRaw());
  });
}

__attribute__((visibility("default"))) int refl_host_tensor_free(void *handle)
{
  return guarded([&] { delete static_cast<CAIF_DeviceTensor *>(handle); });
}

// kind 0: out = a . b;  1: out = a^T . b;  2: out = a . b^T
__attribute__((visibility("default"))) int refl_host_matmul(int kind, void *a, void *b, void *out)
{
  return guarded([&] {
    CAIF_RunContext ctx;
    const CAIF_DeviceTensor &ta = *static_cast<CAIF_DeviceTensor *>(a);
    const CAIF_DeviceTensor &tb = *static_cast<CAIF_DeviceTensor *>(b);
    CAIF_DeviceTensor &to = *static_cast<CAIF_DeviceTensor *>(out);
    if (kind == 0)
    {
      CAIF_Ops::MatMul(ta, tb, to, ctx);
    }
    else if (kind == 1)
    {
      CAIF_Ops::MatMulTransposeA(ta, tb, to, ctx);
    }
    else
    {
      CAIF_Ops::MatMulTransposeB(ta, tb, to, ctx);
    }
  });
}

__attribute__((visibility("default"))) int refl_destroy(void *handle)
{
  return guarded([&] { delete static_cast<Box *>(handle); });
}

__attribute__((visibility("default"))) int refl_moe_layer_create(void *const *experts, uint32_t num_experts,
                                                                 uint32_t input_dim, uint32_t hidden_dim,
                                                                 uint32_t top_k, int storage, int compute,
                                                                 const void *router_w, const void *router_b,
                                                                 int gating_kind, int norm_topk, float scaling,
                                                                 float balance_w, float z_w, void **handle)
{
  return guarded([&] {
    auto box = std::make_unique<Box>();
    const Dtype_e sd = static_cast<Dtype_e>(storage);
    const Dtype_e cd = static_cast<Dtype_e>(compute);
    if (sd == Dtype_e::Float32 && cd == Dtype_e::Float32)
    {
      box->layer = make_moe_layer<float, float>(experts, num_experts, input_dim, hidden_dim, top_k, router_w,
                                                router_b, gating_kind, norm_topk, scaling, balance_w, z_w);
    }
    else if (sd == Dtype_e::BFloat16 && cd == Dtype_e::BFloat16)
    {
      box->layer = make_moe_layer<__nv_bfloat16, __nv_bfloat16>(experts, num_experts, input_dim, hidden_dim, top_k,
                                                                router_w, router_b, gating_kind, norm_topk, scaling,
                                                                balance_w, z_w);
    }
    else
    {
      throw std::runtime_error("moe layer: built for fp32/fp32 and bf16/bf16 only");
    }
    *handle = box.release();
  });
}

// balance and z loss of the last forward pass (LastBalanceLoss / LastZLoss)
__attribute__((visibility("default"))) int refl_moe_layer_losses(void *handle, float *balance, float *z)
{
  return guarded([&] {
    Box *box = static_cast<Box *>(handle);
    if (auto *a = dynamic_cast<CAIF_DeviceMoELayer<float, float> *>(box->layer.get()))
    {
      *balance = a->LastBalanceLoss();
      *z = a->LastZLoss();
    }
    else if (auto *b = dynamic_cast<CAIF_DeviceMoELayer<__nv_bfloat16, __nv_bfloat16> *>(box->layer.get()))
    {
      *balance = b->LastBalanceLoss();
      *z = b->LastZLoss();
    }
    else
    {
      throw std::runtime_error("handle is not a MoE layer");
    }
  });
}

// ---- the reference's SafeTensors reader / writer and name mapper -------------------------------
// Lists come back as '\n'-joined text in the caller's buffer.  TensorInfos, Metadata and the mapper touch
// no device; Save and Load go through CAIF_DeviceTensor::FromHostRaw / CopyToHostRaw.
static void refl_text_out(const std::string &text, char *buf, size_t cap)
{
  if (text.size() + 1 > cap)
  {
    throw std::runtime_error("caller buffer too small");
  }
  std::memcpy(buf, text.c_str(), text.size() + 1);
}

static std::vector<std::string> refl_lines(const char *text)
{
  std::vector<std::string> out;
  std::string cur;
  for (const char *p = text; p != nullptr && *p != '\0'; ++p)
  {
    if (*p == '\n')
    {
      out.push_back(cur);
      cur.clear();
    }
    else
    {
      cur += *p;
    }
  }
  if (!cur.empty())
  {
    out.push_back(cur);
  }
  return out;
}

// one line per tensor, sorted by name: name '\t' dtype '\t' d0,d1,... '\t' begin '\t' end
__attribute__((visibility("default"))) int refl_st_tensor_infos(const char *path, char *buf, size_t cap)
{
  return guarded([&] {
    CAIF_SafeTensorsFormat fmt;
    std::string text;
    for (const auto &kv : fmt.TensorInfos(path))
    {
      text += kv.first + "\t" + kv.second.dtype + "\t";
      for (size_t i = 0; i < kv.second.shape.size(); ++i)
      {
        text += (i ? "," : "") + std::to_string(kv.second.shape[i]);
      }
      text += "\t" + std::to_string(kv.second.data_offset_start) + "\t" + std::to_string(kv.second.data_offset_end) + "\n";
    }
    refl_text_out(text, buf, cap);
  });
}

__attribute__((visibility("default"))) int refl_st_metadata(const char *path, char *buf, size_t cap)
{
  return guarded([&] {
    CAIF_SafeTensorsFormat fmt;
    std::string text;
    for (const auto &kv : fmt.Metadata(path))
    {
      text += kv.first + "\n" + kv.second + "\n";
    }
    refl_text_out(text, buf, cap);
  });
}

__attribute__((visibility("default"))) int refl_st_save(const char *path, uint32_t count, const char *const *names,
                                                        const int *dtypes, const uint32_t *ranks,
                                                        const uint32_t *shapes, const void *const *host_data,
                                                        uint32_t meta_count, const char *const *meta_keys,
                                                        const char *const *meta_values)
{
  return guarded([&] {
    std::vector<CAIF_DeviceTensor> held;
    held.reserve(count);
    const uint32_t *dim = shapes;
    for (uint32_t i = 0; i < count; ++i)
    {
      held.push_back(CAIF_DeviceTensor::FromHostRaw(host_data[i], std::vector<uint32_t>(dim, dim + ranks[i]), stream(),
                                                    static_cast<Dtype_e>(dtypes[i])));
      dim += ranks[i];
    }
    stream().Synchronize();
    std::vector<std::pair<std::string, const CAIF_DeviceTensor *>> list;
    for (uint32_t i = 0; i < count; ++i)
    {
      list.emplace_back(names[i], &held[i]);
    }
    std::map<std::string, std::string> meta;
    for (uint32_t i = 0; i < meta_count; ++i)
    {
      meta[meta_keys[i]] = meta_values[i];
    }
    CAIF_SafeTensorsFormat().Save(path, list, meta);
  });
}

// path: a file, or a checkpoint directory when from_directory != 0 (LoadTensorByName)
__attribute__((visibility("default"))) int refl_st_load(const char *path, int from_directory, const char *name,
                                                        void *out, size_t cap, int *dtype, size_t *bytes)
{
  return guarded([&] {
    CAIF_SafeTensorsFormat fmt;
    CAIF_DeviceTensor t;
    if (from_directory != 0)
    {
      t = fmt.LoadTensorByName(path, name, stream());
    }
    else
    {
      std::map<std::string, CAIF_DeviceTensor> all = fmt.Load(path, stream());
      auto it = all.find(name);
      if (it == all.end())
      {
        throw std::runtime_error("tensor not in file");
      }
      t = std::move(it->second);
    }
    if (t.SizeBytes() > cap)
    {
      throw std::runtime_error("caller buffer too small");
    }
    t.CopyToHostRaw(out);
    stream().Synchronize();
    *dtype = static_cast<int>(t.Dtype());
    *bytes = t.SizeBytes();
  });
}

__attribute__((visibility("default"))) int refl_mapper_create(void **handle)
{
  return guarded([&] { *handle = new CAIF_WeightMapper(); });
}

__attribute__((visibility("default"))) int refl_mapper_destroy(void *handle)
{
  return guarded([&] { delete static_cast<CAIF_WeightMapper *>(handle); });
}

__attribute__((visibility("default"))) int refl_mapper_add(void *handle, int alias, const char *hf, const char *aif)
{
  return guarded([&] {
    auto *m = static_cast<CAIF_WeightMapper *>(handle);
    if (alias != 0)
    {
      m->AddAlias(hf, aif);
    }
    else
    {
      m->AddPrefixRule(hf, aif);
    }
  });
}

__attribute__((visibility("default"))) int refl_mapper_translate(void *handle, int hf_to_aif, const char *name,
                                                                 char *buf, size_t cap)
{
  return guarded([&] {
    auto *m = static_cast<CAIF_WeightMapper *>(handle);
    refl_text_out(hf_to_aif != 0 ? m->HfToAif(name) : m->AifToHf(name), buf, cap);
  });
}

__attribute__((visibility("default"))) int refl_mapper_query(void *handle, int which, const char *aif_names,
                                                             const char *hf_names, char *buf, size_t cap)
{
  return guarded([&] {
    auto *m = static_cast<CAIF_WeightMapper *>(handle);
    const std::vector<std::string> aif = refl_lines(aif_names);
    const std::vector<std::string> hf_list = refl_lines(hf_names);
    const std::set<std::string> hf(hf_list.begin(), hf_list.end());
    std::string text;
    if (which == 0)
    {
      for (const auto &n : m->MissingNames(aif, hf))
      {
        text += n + "\n";
      }
    }
    else if (which == 1)
    {
      for (const auto &n : m->UnmappedHfNames(hf))
      {
        text += n + "\n";
      }
    }
    else
    {
      for (const auto &pr : m->RequiredHfNames(aif))
      {
        text += pr.first + "\n" + pr.second + "\n";
      }
    }
    refl_text_out(text, buf, cap);
  });
}

}  // extern "C"
