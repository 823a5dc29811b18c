// Handle-based C doorway onto the C++ layer classes of caif_host.hpp, so that the
// layer interface (constructor arguments, LoadFromTensor / LoadScalesFromHost,
// Forward / Backward, descriptions, parameter bookkeeping, error behaviour) can
// be driven from a test harness in another language.  Every function returns 0
// on success; after a failure caifh_last_error() holds the exception text.
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "caif_host.hpp"
#include "caif_safetensors.hpp"

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

// ------------------------------------------------------------------ SafeTensors
// One opened file (or checkpoint directory) per handle.  Strings come back in caller buffers; a list
// comes back as its entries joined by '\n'.
namespace
{
struct FileBox
{
  std::unique_ptr<CAIF_SafeTensorsFile> file;
  CAIF_SafeTensorsFormat::ShardedHandle_t directory;
  bool is_directory = false;

  const CAIF_SafeTensorsFile &FileOf(const std::string &name) const
  {
    return is_directory ? directory.ShardOf(name) : *file;
  }
};

std::string joined(const std::vector<std::string> &items)
{
  std::string out;
  for (const std::string &s : items)
  {
    out += s;
    out += '\n';
  }
  return out;
}

std::vector<std::string> split_lines(const char *text)
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

void need_room(const std::string &s, size_t cap)
{
  if (s.size() + 1 > cap)
  {
    THROW_CAIFE("caller buffer too small: " + std::to_string(s.size() + 1) + " bytes needed");
  }
}
}  // namespace

CAIFH_API int caifh_st_open(const char *path, void **handle)
{
  return guarded([&] {
    auto box = std::make_unique<FileBox>();
    box->file = std::make_unique<CAIF_SafeTensorsFile>(path);
    *handle = box.release();
  });
}

// model.safetensors.index.json + shards, or a lone model.safetensors (CAIF_SafeTensorsFormat::OpenShardedHandle)
CAIFH_API int caifh_st_open_directory(const char *directory, void **handle)
{
  return guarded([&] {
    auto box = std::make_unique<FileBox>();
    box->directory = CAIF_SafeTensorsFormat().OpenShardedHandle(directory);
    box->is_directory = true;
    *handle = box.release();
  });
}

CAIFH_API int caifh_st_close(void *handle)
{
  return guarded([&] { delete static_cast<FileBox *>(handle); });
}

// tensor names: a file's in header order, a directory's in weight-map (sorted) order
CAIFH_API int caifh_st_names(void *handle, char *buf, size_t cap)
{
  return guarded([&] {
    auto *box = static_cast<FileBox *>(handle);
    std::vector<std::string> names;
    if (box->is_directory)
    {
      for (const auto &kv : box->directory.WeightMap())
      {
        names.push_back(kv.first);
      }
    }
    else
    {
      names = box->file->NamesInFileOrder();
    }
    const std::string text = joined(names);
    need_room(text, cap);
    copy_string(text, buf, cap);
  });
}

CAIFH_API int caifh_st_info(void *handle, const char *name, char *dtype, size_t dtype_cap, uint32_t *rank,
                            uint32_t *shape, uint32_t shape_cap, uint64_t *begin, uint64_t *end, uint64_t *bytes,
                            char *file_path, size_t file_cap)
{
  return guarded([&] {
    auto *box = static_cast<FileBox *>(handle);
    const CAIF_SafeTensorsFile &file = box->FileOf(name);
    const auto &info = file.Info(name);
    copy_string(info.dtype, dtype, dtype_cap);
    *rank = static_cast<uint32_t>(info.shape.size());
    if (info.shape.size() > shape_cap)
    {
      THROW_CAIFE("shape buffer too small");
    }
    std::copy(info.shape.begin(), info.shape.end(), shape);
    *begin = info.data_offset_start;
    *end = info.data_offset_end;
    *bytes = file.CheckedBytes(info);
    copy_string(file.Path(), file_path, file_cap);
  });
}

// "__metadata__" as key '\n' value '\n' ... (a file only)
CAIFH_API int caifh_st_metadata(void *handle, char *buf, size_t cap)
{
  return guarded([&] {
    auto *box = static_cast<FileBox *>(handle);
    if (box->is_directory)
    {
      THROW_CAIFE("metadata belongs to a file, not a directory");
    }
    std::vector<std::string> flat;
    for (const auto &kv : box->file->Metadata())
    {
      flat.push_back(kv.first);
      flat.push_back(kv.second);
    }
    const std::string text = joined(flat);
    need_room(text, cap);
    copy_string(text, buf, cap);
  });
}

CAIFH_API int caifh_st_read(void *handle, const char *name, void *dst, size_t cap)
{
  return guarded([&] { static_cast<FileBox *>(handle)->FileOf(name).ReadRaw(name, dst, cap); });
}

// Host blobs to a file: dtypes are SafeTensors names, shapes are flattened rank by rank.
CAIFH_API int caifh_st_save(const char *path, uint32_t count, const char *const *names, const char *const *dtypes,
                            const uint32_t *ranks, const uint32_t *shapes, const void *const *data,
                            uint32_t meta_count, const char *const *meta_keys, const char *const *meta_values)
{
  return guarded([&] {
    std::vector<std::pair<std::string, CAIF_SafeTensorsFormat::HostBlob_t>> blobs;
    const uint32_t *dim = shapes;
    for (uint32_t i = 0; i < count; ++i)
    {
      CAIF_SafeTensorsFormat::HostBlob_t blob;
      blob.dtype = dtypes[i];
      blob.shape.assign(dim, dim + ranks[i]);
      dim += ranks[i];
      blob.data = data[i];
      blobs.emplace_back(names[i], std::move(blob));
    }
    std::map<std::string, std::string> meta;
    for (uint32_t i = 0; i < meta_count; ++i)
    {
      meta[meta_keys[i]] = meta_values[i];
    }
    CAIF_SafeTensorsFormat().SaveHost(path, blobs, meta);
  });
}

// Device buffers to a file through CAIF_SafeTensorsFormat::Save (dtypes are CAIF_DataType_e values).
CAIFH_API int caifh_st_save_device(const char *path, uint32_t count, const char *const *names, const int *dtypes,
                                   const uint32_t *ranks, const uint32_t *shapes, void *const *device_data,
                                   void *stream)
{
  return guarded([&] {
    CAIF_CudaStream s(static_cast<cudaStream_t>(stream));
    std::vector<CAIF_DeviceTensor> views;
    views.reserve(count);
    const uint32_t *dim = shapes;
    for (uint32_t i = 0; i < count; ++i)
    {
      views.push_back(CAIF_DeviceTensor::WrapView(device_data[i], std::vector<uint32_t>(dim, dim + ranks[i]), s,
                                                  static_cast<Dtype_e>(dtypes[i])));
      dim += ranks[i];
    }
    std::vector<std::pair<std::string, const CAIF_DeviceTensor *>> list;
    for (uint32_t i = 0; i < count; ++i)
    {
      list.emplace_back(names[i], &views[i]);
    }
    CAIF_SafeTensorsFormat().Save(path, list, {{"framework", "CAIF"}});
  });
}

// A tensor of the file onto the device (native dtype) into caller memory of `cap` bytes.
CAIFH_API int caifh_st_load_device(void *handle, const char *name, void *device_dst, size_t cap, void *stream)
{
  return guarded([&] {
    CAIF_CudaStream s(static_cast<cudaStream_t>(stream));
    CAIF_DeviceTensor t = static_cast<FileBox *>(handle)->FileOf(name).Load(name, s);
    if (t.SizeBytes() > cap)
    {
      THROW_CAIFE("destination too small");
    }
    CAIF_CheckCuda(cudaMemcpyAsync(device_dst, t.DeviceDataRaw(), t.SizeBytes(), cudaMemcpyDeviceToDevice, s.Handle()),
                   "copy");
    CAIF_CheckCuda(cudaStreamSynchronize(s.Handle()), "sync");
  });
}

// LoadFrozenLinear: weight (and scales) of a frozen linear layer straight from a file or directory;
// scales_name may be "" when the stored tensor is a float one.
CAIFH_API int caifh_load_frozen_linear(void *layer_handle, void *st_handle, const char *weight_name,
                                       const char *scales_name)
{
  return guarded([&] {
    auto *box = static_cast<LayerBox *>(layer_handle);
    auto *files = static_cast<FileBox *>(st_handle);
    const CAIF_SafeTensorsFile &file = files->FileOf(weight_name);
    const std::string scales = scales_name != nullptr ? scales_name : "";
    if (!scales.empty() && &files->FileOf(scales) != &file)
    {
      THROW_CAIFE("LoadFrozenLinear: weight and scales must live in the same shard");
    }
    LoadFrozenLinear(*frozen_of(box), file, weight_name, scales, *box->stream);
  });
}

// The layer's trainable tensors to / from a SafeTensors file under ParameterNames(prefix).
CAIFH_API int caifh_save_parameters(void *layer_handle, const char *prefix, const char *path)
{
  return guarded([&] {
    auto *box = static_cast<LayerBox *>(layer_handle);
    SaveParameters(*box->layer, prefix != nullptr ? prefix : "", path, {{"framework", "CAIF"}});
  });
}

CAIFH_API int caifh_load_parameters(void *layer_handle, const char *prefix, void *st_handle)
{
  return guarded([&] {
    auto *box = static_cast<LayerBox *>(layer_handle);
    auto *files = static_cast<FileBox *>(st_handle);
    if (files->is_directory)
    {
      THROW_CAIFE("LoadParameters reads one file");
    }
    LoadParameters(*box->layer, prefix != nullptr ? prefix : "", *files->file, *box->stream);
  });
}

// ------------------------------------------------------------------ name mapping
CAIFH_API int caifh_mapper_create(void **handle)
{
  return guarded([&] { *handle = new CAIF_WeightMapper(); });
}

CAIFH_API int caifh_mapper_destroy(void *handle)
{
  return guarded([&] { delete static_cast<CAIF_WeightMapper *>(handle); });
}

CAIFH_API int caifh_mapper_add(void *handle, int alias, const char *hf, const char *aif)
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

CAIFH_API int caifh_mapper_translate(void *handle, int hf_to_aif, const char *name, char *buf, size_t cap)
{
  return guarded([&] {
    auto *m = static_cast<CAIF_WeightMapper *>(handle);
    const std::string out = hf_to_aif != 0 ? m->HfToAif(name) : m->AifToHf(name);
    need_room(out, cap);
    copy_string(out, buf, cap);
  });
}

// which: 0 MissingNames(aif names, available hf names), 1 UnmappedHfNames(available hf names),
// 2 RequiredHfNames(aif names) as hf '\n' aif pairs.  Lists are '\n'-joined.
CAIFH_API int caifh_mapper_query(void *handle, int which, const char *aif_names, const char *hf_names, char *buf,
                                 size_t cap)
{
  return guarded([&] {
    auto *m = static_cast<CAIF_WeightMapper *>(handle);
    const std::vector<std::string> aif = split_lines(aif_names);
    const std::vector<std::string> hf_list = split_lines(hf_names);
    const std::set<std::string> hf(hf_list.begin(), hf_list.end());
    std::vector<std::string> out;
    if (which == 0)
    {
      out = m->MissingNames(aif, hf);
    }
    else if (which == 1)
    {
      out = m->UnmappedHfNames(hf);
    }
    else
    {
      for (const auto &pair : m->RequiredHfNames(aif))
      {
        out.push_back(pair.first);
        out.push_back(pair.second);
      }
    }
    const std::string text = joined(out);
    need_room(text, cap);
    copy_string(text, buf, cap);
  });
}
