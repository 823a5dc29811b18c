// Handle-based C doorway onto the C++ layer classes of caif_host.hpp, so that the
// layer interface (constructor arguments, LoadFromTensor / LoadScalesFromHost,
// Forward / Backward, descriptions, parameter bookkeeping, error behaviour) can
// be driven from a test harness in another language.  Every function returns 0
// on success; after a failure caifh_last_error() holds the exception text.
#include <cstring>
#include <memory>
#include <string>

#include "caif_host.hpp"

using namespace instance;
using Dtype_e = CAIF_DataType::CAIF_DataType_e;

#define CAIFH_API extern "C" __attribute__((visibility("default")))

namespace
{
thread_local std::string t_error;

struct LayerBox
{
  std::unique_ptr<CAIF_CudaStream> stream;
  std::unique_ptr<CAIF_DeviceLayer> layer;
  Dtype_e storage = Dtype_e::Float32;  // dtype of the activations the layer expects / returns
  Dtype_e out_dtype = Dtype_e::Float32;
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
}

CAIF_DeviceFrozenLinearBase *frozen_of(LayerBox *box)
{
  auto *f = dynamic_cast<CAIF_DeviceFrozenLinearBase *>(box->layer.get());
  if (f == nullptr)
  {
    THROW_CAIFE("handle is not a frozen linear layer");
  }
  return f;
}

template <typename ComputeT>
std::unique_ptr<CAIF_DeviceLayer> make_lora(Dtype_e sd, const CAIF_DeviceLoRAAdapterConfig &cfg,
                                            std::unique_ptr<CAIF_DeviceLayer> base, CAIF_CudaStream &stream,
                                            uint32_t seed)
{
  switch (sd)
  {
    case Dtype_e::Float32:
      return std::make_unique<CAIF_DeviceLoRAAdapter<ComputeT, float>>(cfg, std::move(base), stream, seed);
    case Dtype_e::Float16:
      return std::make_unique<CAIF_DeviceLoRAAdapter<ComputeT, caif_half_t>>(cfg, std::move(base), stream, seed);
    case Dtype_e::BFloat16:
      return std::make_unique<CAIF_DeviceLoRAAdapter<ComputeT, caif_bfloat16_t>>(cfg, std::move(base), stream, seed);
    default:
      break;
  }
  THROW_CAIFE("LoRAAdapter: storage dtype must be fp32, fp16 or bf16");
}

// Moves the frozen linear out of a handle's box (the box is destroyed); the expert owns it afterwards.
std::unique_ptr<CAIF_DeviceFrozenLinearBase> take_frozen(void *handle)
{
  auto *box = static_cast<LayerBox *>(handle);
  if (box == nullptr)
  {
    return nullptr;
  }
  auto *f = dynamic_cast<CAIF_DeviceFrozenLinearBase *>(box->layer.get());
  if (f == nullptr)
  {
    THROW_CAIFE("handle is not a frozen linear layer");
  }
  box->layer.release();
  delete box;
  return std::unique_ptr<CAIF_DeviceFrozenLinearBase>(f);
}

template <typename ComputeT>
std::unique_ptr<CAIF_DeviceLayer> make_expert(Dtype_e sd, const CAIF_DeviceMoEFrozenExpertConfig &cfg, void *gate,
                                              void *up, void *down, CAIF_CudaStream &stream)
{
  switch (sd)
  {
    case Dtype_e::Float32:
    {
      typename CAIF_DeviceMoEFrozenExpert<ComputeT, float>::FrozenSubLayers_t sub;
      sub.gate = take_frozen(gate);
      sub.up = take_frozen(up);
      sub.down = take_frozen(down);
      return std::make_unique<CAIF_DeviceMoEFrozenExpert<ComputeT, float>>(cfg, std::move(sub), stream);
    }
    case Dtype_e::Float16:
    {
      typename CAIF_DeviceMoEFrozenExpert<ComputeT, caif_half_t>::FrozenSubLayers_t sub;
      sub.gate = take_frozen(gate);
      sub.up = take_frozen(up);
      sub.down = take_frozen(down);
      return std::make_unique<CAIF_DeviceMoEFrozenExpert<ComputeT, caif_half_t>>(cfg, std::move(sub), stream);
    }
    case Dtype_e::BFloat16:
    {
      typename CAIF_DeviceMoEFrozenExpert<ComputeT, caif_bfloat16_t>::FrozenSubLayers_t sub;
      sub.gate = take_frozen(gate);
      sub.up = take_frozen(up);
      sub.down = take_frozen(down);
      return std::make_unique<CAIF_DeviceMoEFrozenExpert<ComputeT, caif_bfloat16_t>>(cfg, std::move(sub), stream);
    }
    default:
      break;
  }
  THROW_CAIFE("MoEFrozenExpert: storage dtype must be fp32, fp16 or bf16");
}

void copy_string(const std::string &s, char *buf, size_t cap)
{
  if (cap == 0)
  {
    return;
  }
  std::strncpy(buf, s.c_str(), cap - 1);
  buf[cap - 1] = '\0';
}
}  // namespace

CAIFH_API const char *caifh_last_error(void) { return t_error.c_str(); }

CAIFH_API int caifh_frozen_linear_create(uint32_t in_dim, uint32_t out_dim, int storage, int compute,
                                         uint32_t group_size, int cache_fp32, int int8_scheme, void *stream,
                                         void **handle)
{
  return guarded([&] {
    auto box = std::make_unique<LayerBox>();
    box->stream = std::make_unique<CAIF_CudaStream>(static_cast<cudaStream_t>(stream));
    box->layer = CAIF_DeviceFrozenLinearFactory::Create(in_dim, out_dim, static_cast<Dtype_e>(storage), *box->stream,
                                                        group_size, cache_fp32 != 0, static_cast<Dtype_e>(compute),
                                                        static_cast<CAIF_Ops::QuantScheme_e>(int8_scheme));
    box->storage = static_cast<Dtype_e>(storage);
    box->out_dtype = Dtype_e::Float32;
    *handle = box.release();
  });
}

// Copies `count` elements of `dtype` from device memory into a tensor the layer then owns
// (LoadFromTensor takes ownership in the reference too).  The nominal shape is [in, out], as the
// reference's tests and examples create it; the layer consumes the buffer as flat [out, in].
CAIFH_API int caifh_load_weight_from_device(void *handle, const void *src, int dtype, uint32_t dim0, uint32_t dim1)
{
  return guarded([&] {
    auto *box = static_cast<LayerBox *>(handle);
    CAIF_DeviceTensor t = CAIF_DeviceTensor::Uninitialized({dim0, dim1}, *box->stream, static_cast<Dtype_e>(dtype));
    t.CopyFromDeviceRaw(src, t.SizeBytes());
    frozen_of(box)->LoadFromTensor(std::move(t));
  });
}

CAIFH_API int caifh_load_scales_from_host(void *handle, const void *data, size_t num_bytes)
{
  return guarded([&] { frozen_of(static_cast<LayerBox *>(handle))->LoadScalesFromHost(data, num_bytes); });
}

CAIFH_API int caifh_lora_wrap(void *base_handle, uint32_t rank, float alpha, int storage, int compute, uint32_t seed,
                              void **handle)
{
  return guarded([&] {
    auto *base = static_cast<LayerBox *>(base_handle);
    CAIF_DeviceFrozenLinearBase *f = frozen_of(base);
    const CAIF_DeviceLoRAAdapterConfig cfg(rank, alpha, f->InputDim(), f->OutputDim());
    auto box = std::make_unique<LayerBox>();
    box->stream = std::move(base->stream);
    std::unique_ptr<CAIF_DeviceLayer> inner = std::move(base->layer);
    const Dtype_e sd = static_cast<Dtype_e>(storage);
    switch (static_cast<Dtype_e>(compute))
    {
      case Dtype_e::Float32:
        box->layer = make_lora<float>(sd, cfg, std::move(inner), *box->stream, seed);
        break;
      case Dtype_e::Float16:
        box->layer = make_lora<caif_half_t>(sd, cfg, std::move(inner), *box->stream, seed);
        break;
      case Dtype_e::BFloat16:
        box->layer = make_lora<caif_bfloat16_t>(sd, cfg, std::move(inner), *box->stream, seed);
        break;
      default:
        THROW_CAIFE("LoRAAdapter: compute dtype must be fp32, fp16 or bf16");
    }
    box->storage = sd;
    box->out_dtype = sd;
    delete base;  // its layer and stream moved into the adapter
    *handle = box.release();
  });
}

// A frozen expert over three frozen-linear handles (gate may be null for the non-gated form).  The
// expert takes ownership of the three layers: their handles must not be used or destroyed afterwards.
CAIFH_API int caifh_moe_frozen_expert_create(void *gate, void *up, void *down, uint32_t input_dim, uint32_t hidden_dim,
                                             int use_gated, int storage, int compute, void *stream, void **handle)
{
  return guarded([&] {
    const CAIF_DeviceMoEFrozenExpertConfig cfg(input_dim, hidden_dim, use_gated != 0);
    auto box = std::make_unique<LayerBox>();
    box->stream = std::make_unique<CAIF_CudaStream>(static_cast<cudaStream_t>(stream));
    const Dtype_e sd = static_cast<Dtype_e>(storage);
    switch (static_cast<Dtype_e>(compute))
    {
      case Dtype_e::Float32:
        box->layer = make_expert<float>(sd, cfg, gate, up, down, *box->stream);
        break;
      case Dtype_e::Float16:
        box->layer = make_expert<caif_half_t>(sd, cfg, gate, up, down, *box->stream);
        break;
      case Dtype_e::BFloat16:
        box->layer = make_expert<caif_bfloat16_t>(sd, cfg, gate, up, down, *box->stream);
        break;
      default:
        THROW_CAIFE("MoEFrozenExpert: compute dtype must be fp32, fp16 or bf16");
    }
    box->storage = sd;
    box->out_dtype = sd;
    *handle = box.release();
  });
}

// Forward / Backward on a [rows, last_dim] tensor that lives in device memory at `x`; the result
// (fp32 for a bare frozen linear, the storage dtype for an adapter) is copied to `out`.
static int run(void *handle, bool backward, const void *x, int x_dtype, uint32_t rows, uint32_t last_dim, void *out,
               size_t out_bytes, int training)
{
  return guarded([&] {
    auto *box = static_cast<LayerBox *>(handle);
    CAIF_DeviceTensor in = CAIF_DeviceTensor::WrapView(const_cast<void *>(x), {rows, last_dim}, *box->stream,
                                                       static_cast<Dtype_e>(x_dtype));
    CAIF_RunContext ctx(*box->stream, training != 0);
    CAIF_DeviceTensor res = backward ? box->layer->Backward(in, ctx) : box->layer->Forward(in, ctx);
    if (res.SizeBytes() != out_bytes)
    {
      THROW_CAIFE("result has " + std::to_string(res.SizeBytes()) + " bytes, caller expected " +
                  std::to_string(out_bytes));
    }
    CAIF_CheckCuda(cudaMemcpyAsync(out, res.DeviceDataRaw(), out_bytes, cudaMemcpyDeviceToDevice,
                                   box->stream->Handle()),
                   "copy of the result");
    CAIF_CheckCuda(cudaStreamSynchronize(box->stream->Handle()), "sync");
  });
}

CAIFH_API int caifh_forward(void *handle, const void *x, int x_dtype, uint32_t rows, uint32_t last_dim, void *out,
                            size_t out_bytes, int training)
{
  return run(handle, false, x, x_dtype, rows, last_dim, out, out_bytes, training);
}

CAIFH_API int caifh_backward(void *handle, const void *dy, int dy_dtype, uint32_t rows, uint32_t last_dim, void *out,
                             size_t out_bytes)
{
  return run(handle, true, dy, dy_dtype, rows, last_dim, out, out_bytes, 1);
}

CAIFH_API int caifh_description(void *handle, char *buf, size_t cap)
{
  return guarded([&] { copy_string(static_cast<LayerBox *>(handle)->layer->Description(), buf, cap); });
}

CAIFH_API int caifh_parameter_names(void *handle, const char *prefix, char *buf, size_t cap)
{
  return guarded([&] {
    std::string joined;
    for (const std::string &n : static_cast<LayerBox *>(handle)->layer->ParameterNames(prefix))
    {
      joined += n + ";";
    }
    copy_string(joined, buf, cap);
  });
}

CAIFH_API int caifh_counts(void *handle, uint64_t *param_tensors, uint64_t *total_params, uint64_t *frozen_tensors)
{
  return guarded([&] {
    auto *l = static_cast<LayerBox *>(handle)->layer.get();
    *param_tensors = l->ParameterTensorCount();
    *total_params = l->TotalParameterCount();
    *frozen_tensors = l->FrozenTensorCount();
  });
}

// device-to-device copy of parameter / gradient tensor `index` into or out of the layer
CAIFH_API int caifh_parameter_copy(void *handle, uint64_t index, int gradient, int to_layer, void *buf, size_t bytes)
{
  return guarded([&] {
    auto *box = static_cast<LayerBox *>(handle);
    CAIF_DeviceTensor &t = gradient ? box->layer->GradientTensor(index) : box->layer->ParameterTensor(index);
    if (t.SizeBytes() != bytes)
    {
      THROW_CAIFE("parameter tensor has " + std::to_string(t.SizeBytes()) + " bytes");
    }
    if (to_layer)
    {
      t.CopyFromDeviceRaw(buf, bytes);
    }
    else
    {
      CAIF_CheckCuda(cudaMemcpyAsync(buf, t.DeviceDataRaw(), bytes, cudaMemcpyDeviceToDevice, box->stream->Handle()),
                     "parameter copy");
    }
    CAIF_CheckCuda(cudaStreamSynchronize(box->stream->Handle()), "sync");
  });
}

CAIFH_API int caifh_frozen_tensor_fp32(void *handle, void *out, size_t out_bytes)
{
  return guarded([&] {
    auto *box = static_cast<LayerBox *>(handle);
    CAIF_DeviceTensor t = box->layer->FrozenTensorFP32(0);
    if (t.SizeBytes() != out_bytes)
    {
      THROW_CAIFE("frozen tensor size mismatch");
    }
    CAIF_CheckCuda(cudaMemcpyAsync(out, t.DeviceDataRaw(), out_bytes, cudaMemcpyDeviceToDevice,
                                   box->stream->Handle()),
                   "frozen tensor copy");
    CAIF_CheckCuda(cudaStreamSynchronize(box->stream->Handle()), "sync");
  });
}

CAIFH_API int caifh_destroy(void *handle)
{
  return guarded([&] { delete static_cast<LayerBox *>(handle); });
}
