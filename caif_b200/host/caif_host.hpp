// Host-side layer classes of the quantized frozen-linear path, with the names,
// constructor arguments, accessors and error behaviour of the reference's
// classes, implemented over the C ABI of libcaifq.so (include/caifq.h).
//
//   instance::CAIF_DeviceFrozenLinear<ComputeT,StorageT>   include/caif/caif_device_frozen_linear.h:74-230
//   instance::CAIF_DeviceFrozenLinearBase                  include/caif/caif_device_frozen_linear_base.h:45-80
//   instance::CAIF_DeviceFrozenLinearFactory               include/caif/caif_device_frozen_linear_factory.h:49-59
//   instance::CAIF_DeviceLoRAAdapter<ComputeT,StorageT>    include/caif/caif_device_lora_adapter.h:44-159
//   instance::CAIF_DeviceMoEFrozenExpert<ComputeT,StorageT> include/caif/caif_device_moe_frozen_expert.h:56-174
//
// The reference's tensor / stream / context runtime is out of scope; the small
// vocabulary below (CAIF_DeviceTensor, CAIF_CudaStream, CAIF_RunContext,
// CAIF_DeviceLayer) carries only what these layers touch, with the same
// ownership rules: tensors are move-only, LoadFromTensor takes ownership,
// Forward/Backward return owning tensors, inputs are borrowed.
//
// Differences from the reference that a caller can observe:
//   * no fp32 copy of the weight is cached: CacheFP32() still reports the
//     constructor flag and ClearFP32Cache() is a no-op;
//   * the offload surface (SetOffloadPolicy / Prefetch / Evict) is accepted and
//     ignored: the weight stays resident.
#pragma once

#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdint>
#include <cstring>
#include <ctime>
#include <memory>
#include <random>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "caifq.h"

namespace instance
{

// ------------------------------------------------------------------ vocabulary
class CAIF_Exception : public std::runtime_error
{
  public:
    explicit CAIF_Exception(const std::string &what) : std::runtime_error(what) {}
};

#define THROW_CAIFE(msg) throw ::instance::CAIF_Exception(std::string(msg))

struct CAIF_DataType
{
  enum class CAIF_DataType_e : uint8_t
  {
    Float32 = 0,
    Float64 = 1,
    Float16 = 2,
    BFloat16 = 3,
    Int4 = 4,
    Int8 = 5
  };

  static const char *Name(CAIF_DataType_e d)
  {
    switch (d)
    {
      case CAIF_DataType_e::Float32:
        return "fp32";
      case CAIF_DataType_e::Float64:
        return "fp64";
      case CAIF_DataType_e::Float16:
        return "fp16";
      case CAIF_DataType_e::BFloat16:
        return "bf16";
      case CAIF_DataType_e::Int4:
        return "int4";
      case CAIF_DataType_e::Int8:
        return "int8";
    }
    return "unknown";
  }

  // bytes of `count` elements (int4 packs two per byte)
  static size_t Bytes(CAIF_DataType_e d, size_t count)
  {
    switch (d)
    {
      case CAIF_DataType_e::Float32:
        return count * 4;
      case CAIF_DataType_e::Float64:
        return count * 8;
      case CAIF_DataType_e::Float16:
      case CAIF_DataType_e::BFloat16:
        return count * 2;
      case CAIF_DataType_e::Int4:
        return (count + 1) / 2;
      case CAIF_DataType_e::Int8:
        return count;
    }
    return 0;
  }
};

// storage tag types (the reference uses __half / __nv_bfloat16 / int8_t / caif_int4_packed_t)
struct caif_half_t
{
  uint16_t bits;
};
struct caif_bfloat16_t
{
  uint16_t bits;
};
struct caif_int4_packed_t
{
  uint8_t packed;
};

template <typename T>
struct CAIF_DtypeOf;
template <>
struct CAIF_DtypeOf<float>
{
  static constexpr CAIF_DataType::CAIF_DataType_e value = CAIF_DataType::CAIF_DataType_e::Float32;
};
template <>
struct CAIF_DtypeOf<caif_half_t>
{
  static constexpr CAIF_DataType::CAIF_DataType_e value = CAIF_DataType::CAIF_DataType_e::Float16;
};
template <>
struct CAIF_DtypeOf<caif_bfloat16_t>
{
  static constexpr CAIF_DataType::CAIF_DataType_e value = CAIF_DataType::CAIF_DataType_e::BFloat16;
};
template <>
struct CAIF_DtypeOf<int8_t>
{
  static constexpr CAIF_DataType::CAIF_DataType_e value = CAIF_DataType::CAIF_DataType_e::Int8;
};
template <>
struct CAIF_DtypeOf<caif_int4_packed_t>
{
  static constexpr CAIF_DataType::CAIF_DataType_e value = CAIF_DataType::CAIF_DataType_e::Int4;
};

inline void CAIF_CheckCuda(cudaError_t e, const char *what)
{
  if (e != cudaSuccess)
  {
    THROW_CAIFE(std::string(what) + ": " + cudaGetErrorString(e));
  }
}

inline void CAIF_CheckCaifq(int rc, const char *what)
{
  if (rc != CAIFQ_OK)
  {
    THROW_CAIFE(std::string(what) + ": " + caifq_last_error());
  }
}

class CAIF_CudaStream
{
  public:
    CAIF_CudaStream() : _handle(nullptr) {}
    explicit CAIF_CudaStream(cudaStream_t handle) : _handle(handle) {}
    cudaStream_t Handle() const { return _handle; }

  private:
    cudaStream_t _handle;
};

// Move-only device buffer with a shape and a dtype; owning, or a non-owning view.
class CAIF_DeviceTensor
{
  public:
    using Dtype_e = CAIF_DataType::CAIF_DataType_e;

    CAIF_DeviceTensor() = default;
    CAIF_DeviceTensor(const CAIF_DeviceTensor &) = delete;
    CAIF_DeviceTensor &operator=(const CAIF_DeviceTensor &) = delete;
    CAIF_DeviceTensor(CAIF_DeviceTensor &&o) noexcept { MoveFrom(o); }
    CAIF_DeviceTensor &operator=(CAIF_DeviceTensor &&o) noexcept
    {
      if (this != &o)
      {
        Release();
        MoveFrom(o);
      }
      return *this;
    }
    ~CAIF_DeviceTensor() { Release(); }

    static CAIF_DeviceTensor Uninitialized(const std::vector<uint32_t> &shape, const CAIF_CudaStream &stream,
                                           Dtype_e dtype = Dtype_e::Float32)
    {
      CAIF_DeviceTensor t;
      t._shape = shape;
      t._dtype = dtype;
      t._stream = stream.Handle();
      t._owns = true;
      const size_t bytes = t.SizeBytes();
      if (bytes > 0)
      {
        // stream-ordered allocation from the device's pool: no device-wide synchronisation, and a
        // temporary can be released while the kernels that use it are still queued on the stream
        CAIF_CheckCuda(cudaMallocAsync(&t._data, bytes, t._stream), "CAIF_DeviceTensor: cudaMallocAsync");
      }
      return t;
    }

    static CAIF_DeviceTensor Zeros(const std::vector<uint32_t> &shape, const CAIF_CudaStream &stream,
                                   Dtype_e dtype = Dtype_e::Float32)
    {
      CAIF_DeviceTensor t = Uninitialized(shape, stream, dtype);
      if (t.SizeBytes() > 0)
      {
        CAIF_CheckCuda(cudaMemsetAsync(t._data, 0, t.SizeBytes(), stream.Handle()), "CAIF_DeviceTensor: memset");
      }
      return t;
    }

    static CAIF_DeviceTensor WrapView(void *data, const std::vector<uint32_t> &shape, const CAIF_CudaStream &stream,
                                      Dtype_e dtype)
    {
      CAIF_DeviceTensor t;
      t._shape = shape;
      t._dtype = dtype;
      t._stream = stream.Handle();
      t._data = data;
      t._owns = false;
      return t;
    }

    bool IsAllocated() const { return _data != nullptr; }
    bool IsEmpty() const { return _data == nullptr || NumElements() == 0; }
    const std::vector<uint32_t> &Shape() const { return _shape; }
    Dtype_e Dtype() const { return _dtype; }
    void *DeviceDataRaw() { return _data; }
    const void *DeviceDataRaw() const { return _data; }

    size_t NumElements() const
    {
      size_t n = _shape.empty() ? 0 : 1;
      for (uint32_t d : _shape)
      {
        n *= d;
      }
      return n;
    }
    size_t SizeBytes() const { return CAIF_DataType::Bytes(_dtype, NumElements()); }

    void Reshape(const std::vector<uint32_t> &shape)
    {
      size_t n = shape.empty() ? 0 : 1;
      for (uint32_t d : shape)
      {
        n *= d;
      }
      if (n != NumElements())
      {
        THROW_CAIFE("CAIF_DeviceTensor::Reshape: element count mismatch");
      }
      _shape = shape;
    }

    void CopyFromHostRaw(const void *src, size_t bytes)
    {
      if (bytes > SizeBytes())
      {
        THROW_CAIFE("CAIF_DeviceTensor::CopyFromHostRaw: source larger than the tensor");
      }
      CAIF_CheckCuda(cudaMemcpyAsync(_data, src, bytes, cudaMemcpyHostToDevice, _stream), "CopyFromHostRaw");
      CAIF_CheckCuda(cudaStreamSynchronize(_stream), "CopyFromHostRaw: sync");
    }

    void CopyToHostRaw(void *dst) const
    {
      CAIF_CheckCuda(cudaMemcpyAsync(dst, _data, SizeBytes(), cudaMemcpyDeviceToHost, _stream), "CopyToHostRaw");
      CAIF_CheckCuda(cudaStreamSynchronize(_stream), "CopyToHostRaw: sync");
    }

    void CopyFromDeviceRaw(const void *src, size_t bytes)
    {
      if (bytes > SizeBytes())
      {
        THROW_CAIFE("CAIF_DeviceTensor::CopyFromDeviceRaw: source larger than the tensor");
      }
      CAIF_CheckCuda(cudaMemcpyAsync(_data, src, bytes, cudaMemcpyDeviceToDevice, _stream), "CopyFromDeviceRaw");
    }

  private:
    void Release()
    {
      if (_owns && _data != nullptr)
      {
        cudaFreeAsync(_data, _stream);   // ordered behind everything queued on the tensor's stream
      }
      _data = nullptr;
    }
    void MoveFrom(CAIF_DeviceTensor &o)
    {
      _data = o._data;
      _shape = std::move(o._shape);
      _dtype = o._dtype;
      _stream = o._stream;
      _owns = o._owns;
      o._data = nullptr;
      o._owns = false;
      o._shape.clear();
    }

    void *_data = nullptr;
    std::vector<uint32_t> _shape;
    Dtype_e _dtype = Dtype_e::Float32;
    cudaStream_t _stream = nullptr;
    bool _owns = false;
};

class CAIF_RunContext
{
  public:
    enum class Subsystem_e : uint8_t
    {
      None_e,
      FrozenLinear_e,
      LoRAAdapter_e,
      MoEFrozenExpert_e
    };
    CAIF_RunContext(CAIF_CudaStream &stream, bool training) : _stream(&stream), _training(training) {}
    bool Training() const { return _training; }
    void SetTraining(bool t) { _training = t; }
    CAIF_CudaStream &Stream() { return *_stream; }
    void PushSubsystem(Subsystem_e s) { _stack.push_back(s); }
    void PopSubsystem() { _stack.pop_back(); }
    Subsystem_e CurrentSubsystem() const { return _stack.empty() ? Subsystem_e::None_e : _stack.back(); }

  private:
    CAIF_CudaStream *_stream;
    bool _training;
    std::vector<Subsystem_e> _stack;
};

struct CAIF_Ops
{
  enum class QuantScheme_e : uint8_t
  {
    PerTensor_e,
    PerChannel_e
  };
};

struct CAIF_OffloadPolicy
{
  enum class CAIF_OffloadPolicy_e : uint8_t
  {
    GpuResident_e,
    HostPinned_e
  };
};

constexpr uint32_t g_caif_quant_default_group_size = 128;

// The dtype-erased layer root (include/caif/caif_device_layer.h:83-195): Forward/Backward push
// the subsystem tag and call the Impl.
class CAIF_DeviceLayer
{
  public:
    explicit CAIF_DeviceLayer(CAIF_CudaStream &stream) : _stream(&stream) {}
    virtual ~CAIF_DeviceLayer() = default;

    CAIF_DeviceTensor Forward(const CAIF_DeviceTensor &input, CAIF_RunContext &ctx)
    {
      ctx.PushSubsystem(SubsystemTag());
      struct Pop
      {
        CAIF_RunContext &c;
        ~Pop() { c.PopSubsystem(); }
      } pop{ctx};
      return ForwardImpl(input, ctx);
    }
    CAIF_DeviceTensor Backward(const CAIF_DeviceTensor &grad_output, CAIF_RunContext &ctx)
    {
      ctx.PushSubsystem(SubsystemTag());
      struct Pop
      {
        CAIF_RunContext &c;
        ~Pop() { c.PopSubsystem(); }
      } pop{ctx};
      return BackwardImpl(grad_output, ctx);
    }

    virtual CAIF_DeviceTensor ForwardImpl(const CAIF_DeviceTensor &input, CAIF_RunContext &ctx) = 0;
    virtual CAIF_DeviceTensor BackwardImpl(const CAIF_DeviceTensor &grad_output, CAIF_RunContext &ctx) = 0;
    virtual CAIF_RunContext::Subsystem_e SubsystemTag() const = 0;
    virtual void ZeroGradients() = 0;
    virtual size_t ParameterTensorCount() const = 0;
    virtual CAIF_DeviceTensor &ParameterTensor(size_t index) = 0;
    virtual CAIF_DeviceTensor &GradientTensor(size_t index) = 0;
    virtual size_t TotalParameterCount() const = 0;
    virtual std::string Description() const = 0;
    virtual std::vector<std::string> ParameterNames(const std::string &prefix = "") const = 0;
    virtual size_t FrozenTensorCount() const { return 0; }
    virtual CAIF_DeviceTensor FrozenTensorFP32(size_t) const { THROW_CAIFE("layer has no frozen tensors"); }
    virtual std::vector<std::string> FrozenTensorNames(const std::string & = "") const { return {}; }

    bool HasStream() const { return _stream != nullptr; }
    CAIF_CudaStream &Stream() const { return *_stream; }

  private:
    CAIF_CudaStream *_stream;
};

template <typename ComputeT, typename StorageT>
class CAIF_DeviceLayerTyped : public CAIF_DeviceLayer
{
  public:
    explicit CAIF_DeviceLayerTyped(CAIF_CudaStream &stream) : CAIF_DeviceLayer(stream) {}
    static constexpr CAIF_DataType::CAIF_DataType_e StorageDtype() { return CAIF_DtypeOf<StorageT>::value; }
    static constexpr CAIF_DataType::CAIF_DataType_e ComputeDtype() { return CAIF_DtypeOf<ComputeT>::value; }
};

// ------------------------------------------------------------------ frozen linear
class CAIF_DeviceFrozenLinearBase
{
  public:
    virtual ~CAIF_DeviceFrozenLinearBase() = default;
    virtual void LoadFromTensor(CAIF_DeviceTensor &&weight) = 0;
    virtual void LoadScalesFromHost(const void *data, size_t num_bytes) = 0;
    virtual void ClearFP32Cache() = 0;
    virtual bool NeedsScales() const = 0;
    virtual CAIF_Ops::QuantScheme_e Int8Scheme() const = 0;
    virtual bool CacheFP32() const = 0;
    virtual uint32_t InputDim() const = 0;
    virtual uint32_t OutputDim() const = 0;
    // what a loader needs before any weight is loaded: the stored dtype and the int4 group length
    virtual CAIF_DataType::CAIF_DataType_e WeightStorageDtype() const = 0;
    virtual uint32_t QuantGroupSize() const = 0;
    virtual void SetOffloadPolicy(const CAIF_OffloadPolicy::CAIF_OffloadPolicy_e) {}
    virtual CAIF_OffloadPolicy::CAIF_OffloadPolicy_e OffloadPolicy() const
    {
      return CAIF_OffloadPolicy::CAIF_OffloadPolicy_e::GpuResident_e;
    }
    virtual void Prefetch(CAIF_CudaStream &) {}
    virtual void Evict() {}
    virtual bool IsPrefetched() const { return true; }
    // the C-ABI view of the stored weight (what the fused LoRA / expert paths consume)
    virtual caifq_weight AsCaifqWeight() const = 0;
};

template <typename ComputeT = float, typename StorageT = float>
class CAIF_DeviceFrozenLinear : public CAIF_DeviceLayerTyped<ComputeT, StorageT>, public CAIF_DeviceFrozenLinearBase
{
  public:
    typedef CAIF_DeviceLayerTyped<ComputeT, StorageT> Base_t;
    using Base_t::HasStream;
    using Base_t::Stream;
    using Dtype_e = CAIF_DataType::CAIF_DataType_e;

    CAIF_DeviceFrozenLinear(uint32_t input_dim, uint32_t output_dim, CAIF_CudaStream &stream,
                            uint32_t group_size = g_caif_quant_default_group_size, bool cache_fp32 = true,
                            CAIF_Ops::QuantScheme_e int8_scheme = CAIF_Ops::QuantScheme_e::PerTensor_e)
        : Base_t(stream),
          _input_dim(input_dim),
          _output_dim(output_dim),
          _group_size(group_size),
          _cache_fp32(cache_fp32),
          _int8_scheme(int8_scheme)
    {
      if (input_dim == 0 || output_dim == 0)
      {
        THROW_CAIFE("FrozenLinear: input_dim and output_dim must be > 0");
      }
    }

    // ---- CAIF_DeviceLayer ------------------------------------------------------
    CAIF_DeviceTensor ForwardImpl(const CAIF_DeviceTensor &input, CAIF_RunContext &ctx) override
    {
      const uint32_t n = CheckedRows(input, _input_dim, "FrozenLinear::Forward");
      if (ctx.Training())
      {
        _forward_ran = true;  // the reference keeps a clone of the input only as this flag (:437-440, :543-546)
      }
      std::vector<uint32_t> out_shape(input.Shape().begin(), input.Shape().end() - 1);
      out_shape.push_back(_output_dim);
      CAIF_DeviceTensor output = CAIF_DeviceTensor::Uninitialized(out_shape, Stream());  // fp32, always
      const caifq_weight w = AsCaifqWeight();
      CAIF_CheckCaifq(caifq_linear_fwd(&w, input.DeviceDataRaw(), static_cast<int32_t>(input.Dtype()), n,
                                       output.DeviceDataRaw(), CAIFQ_F32,
                                       static_cast<int32_t>(Base_t::ComputeDtype()), Stream().Handle()),
                      "FrozenLinear::Forward");
      return output;
    }

    CAIF_DeviceTensor BackwardImpl(const CAIF_DeviceTensor &grad_output, CAIF_RunContext &) override
    {
      if (!_forward_ran)
      {
        THROW_CAIFE("FrozenLinear::Backward: must call Forward(training=true) first");
      }
      const uint32_t n = CheckedRows(grad_output, _output_dim, "FrozenLinear::Backward");
      std::vector<uint32_t> in_shape(grad_output.Shape().begin(), grad_output.Shape().end() - 1);
      in_shape.push_back(_input_dim);
      CAIF_DeviceTensor grad_input = CAIF_DeviceTensor::Uninitialized(in_shape, Stream());
      const caifq_weight w = AsCaifqWeight();
      CAIF_CheckCaifq(caifq_linear_dx(&w, grad_output.DeviceDataRaw(), static_cast<int32_t>(grad_output.Dtype()), n,
                                      grad_input.DeviceDataRaw(), CAIFQ_F32,
                                      static_cast<int32_t>(Base_t::ComputeDtype()), Stream().Handle()),
                      "FrozenLinear::Backward");
      return grad_input;
    }

    CAIF_RunContext::Subsystem_e SubsystemTag() const override { return CAIF_RunContext::Subsystem_e::FrozenLinear_e; }
    void ZeroGradients() override {}
    size_t ParameterTensorCount() const override { return 0; }
    CAIF_DeviceTensor &ParameterTensor(size_t) override { THROW_CAIFE("FrozenLinear: no trainable parameters"); }
    CAIF_DeviceTensor &GradientTensor(size_t) override { THROW_CAIFE("FrozenLinear: no trainable parameters"); }
    size_t TotalParameterCount() const override { return 0; }
    std::string Description() const override
    {
      return std::string("FrozenLinear(") + std::to_string(_input_dim) + "," + std::to_string(_output_dim) + "," +
             CAIF_DataType::Name(Base_t::StorageDtype()) + ")";
    }
    std::vector<std::string> ParameterNames(const std::string & = "") const override { return {}; }
    size_t FrozenTensorCount() const override { return 1; }
    CAIF_DeviceTensor FrozenTensorFP32(size_t index) const override
    {
      if (index != 0)
      {
        THROW_CAIFE("FrozenLinear: frozen tensor index out of range");
      }
      const caifq_weight w = AsCaifqWeight();
      CAIF_DeviceTensor fp32 = CAIF_DeviceTensor::Uninitialized({_output_dim, _input_dim}, Stream());
      CAIF_CheckCaifq(caifq_weight_materialize(&w, fp32.DeviceDataRaw(), CAIFQ_F32, Stream().Handle()),
                      "FrozenLinear::FrozenTensorFP32");
      return fp32;
    }
    std::vector<std::string> FrozenTensorNames(const std::string &prefix = "") const override
    {
      return {prefix + "weight"};
    }

    // ---- CAIF_DeviceFrozenLinearBase --------------------------------------------
    void LoadFromTensor(CAIF_DeviceTensor &&weight) override
    {
      // the buffer is consumed as flat row-major [out, in] whatever nominal shape it carries
      if (weight.NumElements() != static_cast<size_t>(_input_dim) * _output_dim &&
          weight.SizeBytes() != CAIF_DataType::Bytes(Base_t::StorageDtype(), static_cast<size_t>(_input_dim) * _output_dim))
      {
        THROW_CAIFE("FrozenLinear::LoadFromTensor: element count does not match input_dim*output_dim");
      }
      _weight = std::move(weight);
    }

    void LoadScalesFromHost(const void *data, size_t num_bytes) override
    {
      constexpr Dtype_e sd = Base_t::StorageDtype();
      if (sd == Dtype_e::Int4)
      {
        const size_t total = static_cast<size_t>(_input_dim) * _output_dim;
        const uint32_t groups = static_cast<uint32_t>((total + _group_size - 1) / _group_size);
        _scales = CAIF_DeviceTensor::Zeros({groups}, Stream(), Dtype_e::Float16);
        _scales.CopyFromHostRaw(data, num_bytes);
        return;
      }
      if (sd == Dtype_e::Int8)
      {
        const uint32_t count = (_int8_scheme == CAIF_Ops::QuantScheme_e::PerTensor_e) ? 1u : _output_dim;
        _scales = CAIF_DeviceTensor::Zeros({count}, Stream(), Dtype_e::Float32);
        _scales.CopyFromHostRaw(data, num_bytes);
        return;
      }
      THROW_CAIFE("FrozenLinear::LoadScalesFromHost: storage dtype does not use scales");
    }

    // scales that already live on the device (what a quantizer on the GPU produced)
    void LoadScalesFromDevice(const void *data, size_t num_bytes)
    {
      constexpr Dtype_e sd = Base_t::StorageDtype();
      if (sd != Dtype_e::Int4 && sd != Dtype_e::Int8)
      {
        THROW_CAIFE("FrozenLinear::LoadScalesFromDevice: storage dtype does not use scales");
      }
      const Dtype_e dt = (sd == Dtype_e::Int4) ? Dtype_e::Float16 : Dtype_e::Float32;
      const uint32_t count = static_cast<uint32_t>(num_bytes / CAIF_DataType::Bytes(dt, 1));
      _scales = CAIF_DeviceTensor::Uninitialized({count}, Stream(), dt);
      _scales.CopyFromDeviceRaw(data, num_bytes);
    }

    void ClearFP32Cache() override {}
    bool NeedsScales() const override
    {
      constexpr Dtype_e sd = Base_t::StorageDtype();
      return sd == Dtype_e::Int4 || sd == Dtype_e::Int8;
    }
    CAIF_Ops::QuantScheme_e Int8Scheme() const override { return _int8_scheme; }
    bool CacheFP32() const override { return _cache_fp32; }
    uint32_t InputDim() const override { return _input_dim; }
    uint32_t OutputDim() const override { return _output_dim; }
    uint32_t GroupSize() const { return _group_size; }
    CAIF_DataType::CAIF_DataType_e WeightStorageDtype() const override { return Base_t::StorageDtype(); }
    uint32_t QuantGroupSize() const override { return _group_size; }

    caifq_weight AsCaifqWeight() const override
    {
      if (_weight.IsEmpty())
      {
        THROW_CAIFE("FrozenLinear: weight not loaded");
      }
      caifq_weight w;
      w.codes = _weight.DeviceDataRaw();
      w.scales = _scales.IsEmpty() ? nullptr : _scales.DeviceDataRaw();
      w.storage = static_cast<int32_t>(Base_t::StorageDtype());
      w.scheme = static_cast<int32_t>(_int8_scheme);
      w.group_size = static_cast<int32_t>(_group_size);
      w.in_dim = static_cast<int32_t>(_input_dim);
      w.out_dim = static_cast<int32_t>(_output_dim);
      return w;
    }

  private:
    uint32_t CheckedRows(const CAIF_DeviceTensor &t, uint32_t last_dim, const char *who) const
    {
      if (!HasStream())
      {
        THROW_CAIFE("FrozenLinear: stream is null");
      }
      if (_weight.IsEmpty())
      {
        THROW_CAIFE("FrozenLinear: weight not loaded");
      }
      const auto &shape = t.Shape();
      if (shape.size() < 2)
      {
        THROW_CAIFE(std::string(who) + ": input must be at least 2D");
      }
      if (shape.back() != last_dim)
      {
        THROW_CAIFE(std::string(who) + ": last dim must match the layer");
      }
      uint32_t n = 1;
      for (size_t i = 0; i + 1 < shape.size(); ++i)
      {
        n *= shape[i];
      }
      return n;
    }

    uint32_t _input_dim;
    uint32_t _output_dim;
    uint32_t _group_size;
    bool _cache_fp32;
    CAIF_Ops::QuantScheme_e _int8_scheme;
    CAIF_DeviceTensor _weight;
    CAIF_DeviceTensor _scales;
    bool _forward_ran = false;
};

class CAIF_DeviceFrozenLinearFactory
{
  public:
    CAIF_DeviceFrozenLinearFactory() = delete;
    using Dtype_e = CAIF_DataType::CAIF_DataType_e;

    // the 3 x 5 (compute, storage) grid of src/caif_device_frozen_linear_factory.cpp:46-139
    static std::unique_ptr<CAIF_DeviceLayer> Create(uint32_t input_dim, uint32_t output_dim, Dtype_e storage_dtype,
                                                    CAIF_CudaStream &stream,
                                                    uint32_t group_size = g_caif_quant_default_group_size,
                                                    bool cache_fp32 = true, Dtype_e compute_dtype = Dtype_e::Float32,
                                                    CAIF_Ops::QuantScheme_e int8_scheme =
                                                        CAIF_Ops::QuantScheme_e::PerTensor_e)
    {
      switch (compute_dtype)
      {
        case Dtype_e::Float32:
          return ForCompute<float>(input_dim, output_dim, storage_dtype, stream, group_size, cache_fp32, int8_scheme);
        case Dtype_e::Float16:
          return ForCompute<caif_half_t>(input_dim, output_dim, storage_dtype, stream, group_size, cache_fp32,
                                         int8_scheme);
        case Dtype_e::BFloat16:
          return ForCompute<caif_bfloat16_t>(input_dim, output_dim, storage_dtype, stream, group_size, cache_fp32,
                                             int8_scheme);
        default:
          break;
      }
      THROW_CAIFE("CAIF_DeviceFrozenLinearFactory::Create: unsupported (storage,compute) dtype pair");
    }

  private:
    template <typename ComputeT>
    static std::unique_ptr<CAIF_DeviceLayer> ForCompute(uint32_t in, uint32_t out, Dtype_e storage,
                                                        CAIF_CudaStream &stream, uint32_t group, bool cache,
                                                        CAIF_Ops::QuantScheme_e scheme)
    {
      switch (storage)
      {
        case Dtype_e::Float32:
          return std::make_unique<CAIF_DeviceFrozenLinear<ComputeT, float>>(in, out, stream, group, cache, scheme);
        case Dtype_e::Float16:
          return std::make_unique<CAIF_DeviceFrozenLinear<ComputeT, caif_half_t>>(in, out, stream, group, cache,
                                                                                  scheme);
        case Dtype_e::BFloat16:
          return std::make_unique<CAIF_DeviceFrozenLinear<ComputeT, caif_bfloat16_t>>(in, out, stream, group, cache,
                                                                                      scheme);
        case Dtype_e::Int8:
          return std::make_unique<CAIF_DeviceFrozenLinear<ComputeT, int8_t>>(in, out, stream, group, cache, scheme);
        case Dtype_e::Int4:
          return std::make_unique<CAIF_DeviceFrozenLinear<ComputeT, caif_int4_packed_t>>(in, out, stream, group,
                                                                                         cache, scheme);
        default:
          break;
      }
      THROW_CAIFE("CAIF_DeviceFrozenLinearFactory::Create: unsupported (storage,compute) dtype pair");
    }
};

// ------------------------------------------------------------------ LoRA adapter
class CAIF_DeviceLoRAAdapterConfig
{
  public:
    CAIF_DeviceLoRAAdapterConfig(uint32_t rank, float alpha, uint32_t input_dim, uint32_t output_dim)
        : _rank(rank), _alpha(alpha), _input_dim(input_dim), _output_dim(output_dim)
    {
    }
    uint32_t Rank() const { return _rank; }
    float Alpha() const { return _alpha; }
    uint32_t InputDim() const { return _input_dim; }
    uint32_t OutputDim() const { return _output_dim; }

  private:
    uint32_t _rank;
    float _alpha;
    uint32_t _input_dim;
    uint32_t _output_dim;
};

// fp32 -> storage bits on the host, round to nearest even (what CopyFromHostFp32 does for A's init)
inline uint16_t CAIF_HostFloatToBf16(float f)
{
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u)
  {
    return 0x7FFF;
  }
  x += 0x7FFFu + ((x >> 16) & 1u);
  return static_cast<uint16_t>(x >> 16);
}

template <typename ComputeT = float, typename StorageT = float>
class CAIF_DeviceLoRAAdapter : public CAIF_DeviceLayerTyped<ComputeT, StorageT>
{
  public:
    typedef CAIF_DeviceLayerTyped<ComputeT, StorageT> Base_t;
    using Base_t::Stream;
    using Dtype_e = CAIF_DataType::CAIF_DataType_e;

    // A [rank, in] is Kaiming-uniform U(-sqrt(1/in), +sqrt(1/in)) from std::mt19937(seed)
    // (seed 0 = time), B [out, rank] starts at zero: src/caif_device_lora_adapter.cpp:29-82.
    CAIF_DeviceLoRAAdapter(const CAIF_DeviceLoRAAdapterConfig &config, std::unique_ptr<CAIF_DeviceLayer> base_layer,
                           CAIF_CudaStream &stream, uint32_t seed = 0)
        : Base_t(stream), _config(config), _base_layer(std::move(base_layer))
    {
      if (config.Rank() == 0 || config.InputDim() == 0 || config.OutputDim() == 0)
      {
        THROW_CAIFE("LoRAAdapter: rank, input_dim, output_dim must be > 0");
      }
      if (!_base_layer)
      {
        THROW_CAIFE("LoRAAdapter: base_layer must not be null");
      }
      _frozen = dynamic_cast<CAIF_DeviceFrozenLinearBase *>(_base_layer.get());
      if (_frozen == nullptr)
      {
        THROW_CAIFE("LoRAAdapter: this build adapts frozen linear layers only");
      }
      constexpr Dtype_e sd = Base_t::StorageDtype();
      _lora_a = CAIF_DeviceTensor::Uninitialized({config.Rank(), config.InputDim()}, stream, sd);
      _lora_b = CAIF_DeviceTensor::Zeros({config.OutputDim(), config.Rank()}, stream, sd);
      _grad_lora_a = CAIF_DeviceTensor::Zeros({config.Rank(), config.InputDim()}, stream, sd);
      _grad_lora_b = CAIF_DeviceTensor::Zeros({config.OutputDim(), config.Rank()}, stream, sd);
      if (seed == 0)
      {
        seed = static_cast<uint32_t>(std::time(nullptr));
      }
      const float bound = std::sqrt(1.0f / static_cast<float>(config.InputDim()));
      std::mt19937 gen(seed);
      std::uniform_real_distribution<float> dist(-bound, bound);
      const size_t count = static_cast<size_t>(config.Rank()) * config.InputDim();
      std::vector<float> host_a(count);
      for (size_t i = 0; i < count; ++i)
      {
        host_a[i] = dist(gen);
      }
      UploadFp32(_lora_a, host_a);
    }

    CAIF_DeviceTensor ForwardImpl(const CAIF_DeviceTensor &input, CAIF_RunContext &ctx) override
    {
      const uint32_t n = Rows(input, _config.InputDim(), "LoRAAdapter::Forward");
      constexpr Dtype_e sd = Base_t::StorageDtype();
      if (input.Dtype() != sd)
      {
        THROW_CAIFE("LoRAAdapter::Forward: input dtype must equal the adapter's storage dtype");
      }
      std::vector<uint32_t> out_shape(input.Shape().begin(), input.Shape().end() - 1);
      out_shape.push_back(_config.OutputDim());
      CAIF_DeviceTensor output = CAIF_DeviceTensor::Uninitialized(out_shape, Stream(), sd);
      CAIF_DeviceTensor hidden = CAIF_DeviceTensor::Uninitialized({n, _config.Rank()}, Stream(), sd);
      const caifq_weight w = _frozen->AsCaifqWeight();
      const caifq_lora l = AsCaifqLora();
      // (the entry points that may expand the weight once per call: the layer owns stream-ordered scratch)
      const int32_t cd = static_cast<int32_t>(Base_t::ComputeDtype());
      const size_t ws_bytes = caifq_lora_fwd_workspace_bytes_expanded(&w, &l, n, cd);
      CAIF_DeviceTensor ws =
          CAIF_DeviceTensor::Uninitialized({static_cast<uint32_t>(ws_bytes)}, Stream(), Dtype_e::Int8);
      CAIF_CheckCaifq(caifq_lora_linear_fwd_expanded(&w, &l, input.DeviceDataRaw(), n, output.DeviceDataRaw(),
                                                     hidden.DeviceDataRaw(), ws.DeviceDataRaw(), cd,
                                                     Stream().Handle()),
                      "LoRAAdapter::Forward");
      if (ctx.Training())
      {
        _cached_input = CAIF_DeviceTensor::Uninitialized({n, _config.InputDim()}, Stream(), sd);
        _cached_input.CopyFromDeviceRaw(input.DeviceDataRaw(), input.SizeBytes());
        _cached_lora_hidden = std::move(hidden);
      }
      return output;
    }

    CAIF_DeviceTensor BackwardImpl(const CAIF_DeviceTensor &grad_output, CAIF_RunContext &) override
    {
      if (_cached_input.IsEmpty())
      {
        THROW_CAIFE("LoRAAdapter::Backward: must call Forward with training=true first");
      }
      const uint32_t n = Rows(grad_output, _config.OutputDim(), "LoRAAdapter::Backward");
      constexpr Dtype_e sd = Base_t::StorageDtype();
      std::vector<uint32_t> in_shape(grad_output.Shape().begin(), grad_output.Shape().end() - 1);
      in_shape.push_back(_config.InputDim());
      CAIF_DeviceTensor grad_input = CAIF_DeviceTensor::Uninitialized(in_shape, Stream(), sd);
      const caifq_weight w = _frozen->AsCaifqWeight();
      const caifq_lora l = AsCaifqLora();
      const int32_t cd = static_cast<int32_t>(Base_t::ComputeDtype());
      const size_t ws_bytes = caifq_lora_bwd_workspace_bytes_expanded(&w, &l, n, cd);
      CAIF_DeviceTensor ws =
          CAIF_DeviceTensor::Uninitialized({static_cast<uint32_t>(ws_bytes)}, Stream(), Dtype_e::Int8);
      CAIF_CheckCaifq(caifq_lora_linear_bwd_expanded(&w, &l, grad_output.DeviceDataRaw(),
                                                     _cached_input.DeviceDataRaw(),
                                                     _cached_lora_hidden.DeviceDataRaw(), n,
                                                     grad_input.DeviceDataRaw(), _grad_lora_a.DeviceDataRaw(),
                                                     _grad_lora_b.DeviceDataRaw(), ws.DeviceDataRaw(), cd,
                                                     Stream().Handle()),
                      "LoRAAdapter::Backward");
      // the workspace is freed when `ws` goes out of scope; cudaFree waits for the work that uses it
      return grad_input;
    }

    CAIF_RunContext::Subsystem_e SubsystemTag() const override { return CAIF_RunContext::Subsystem_e::LoRAAdapter_e; }
    void ZeroGradients() override
    {
      CAIF_CheckCuda(cudaMemsetAsync(_grad_lora_a.DeviceDataRaw(), 0, _grad_lora_a.SizeBytes(), Stream().Handle()),
                     "LoRAAdapter::ZeroGradients");
      CAIF_CheckCuda(cudaMemsetAsync(_grad_lora_b.DeviceDataRaw(), 0, _grad_lora_b.SizeBytes(), Stream().Handle()),
                     "LoRAAdapter::ZeroGradients");
      _base_layer->ZeroGradients();
    }
    // parameter order: [base parameters..., A, B]
    size_t ParameterTensorCount() const override { return _base_layer->ParameterTensorCount() + 2; }
    CAIF_DeviceTensor &ParameterTensor(size_t index) override
    {
      const size_t base = _base_layer->ParameterTensorCount();
      if (index < base)
      {
        return _base_layer->ParameterTensor(index);
      }
      if (index == base)
      {
        return _lora_a;
      }
      if (index == base + 1)
      {
        return _lora_b;
      }
      THROW_CAIFE("LoRAAdapter: parameter index out of range");
    }
    CAIF_DeviceTensor &GradientTensor(size_t index) override
    {
      const size_t base = _base_layer->ParameterTensorCount();
      if (index < base)
      {
        return _base_layer->GradientTensor(index);
      }
      if (index == base)
      {
        return _grad_lora_a;
      }
      if (index == base + 1)
      {
        return _grad_lora_b;
      }
      THROW_CAIFE("LoRAAdapter: gradient index out of range");
    }
    size_t TotalParameterCount() const override
    {
      return _base_layer->TotalParameterCount() + _lora_a.NumElements() + _lora_b.NumElements();
    }
    std::string Description() const override
    {
      return std::string("LoRA(rank=") + std::to_string(_config.Rank()) + ",alpha=" +
             std::to_string(static_cast<int>(_config.Alpha())) + "," + std::to_string(_config.InputDim()) + "," +
             std::to_string(_config.OutputDim()) + ")+" + _base_layer->Description();
    }
    std::vector<std::string> ParameterNames(const std::string &prefix = "") const override
    {
      std::vector<std::string> names = _base_layer->ParameterNames(prefix);
      names.push_back(prefix + "lora_a.weight");
      names.push_back(prefix + "lora_b.weight");
      return names;
    }
    size_t FrozenTensorCount() const override { return _base_layer->FrozenTensorCount(); }
    CAIF_DeviceTensor FrozenTensorFP32(size_t i) const override { return _base_layer->FrozenTensorFP32(i); }
    std::vector<std::string> FrozenTensorNames(const std::string &prefix = "") const override
    {
      return _base_layer->FrozenTensorNames(prefix);
    }

    const CAIF_DeviceLoRAAdapterConfig &Config() const { return _config; }
    CAIF_DeviceLayer &BaseLayer() { return *_base_layer; }
    CAIF_DeviceTensor &LoRAA() { return _lora_a; }
    CAIF_DeviceTensor &LoRAB() { return _lora_b; }
    CAIF_DeviceTensor &GradLoRAA() { return _grad_lora_a; }
    CAIF_DeviceTensor &GradLoRAB() { return _grad_lora_b; }

  private:
    caifq_lora AsCaifqLora() const
    {
      caifq_lora l;
      l.a = _lora_a.DeviceDataRaw();
      l.b = _lora_b.DeviceDataRaw();
      l.dtype = static_cast<int32_t>(Base_t::StorageDtype());
      l.rank = static_cast<int32_t>(_config.Rank());
      l.alpha = _config.Alpha();
      return l;
    }

    uint32_t Rows(const CAIF_DeviceTensor &t, uint32_t last_dim, const char *who) const
    {
      const auto &shape = t.Shape();
      if (shape.size() < 2)
      {
        THROW_CAIFE(std::string(who) + ": input must be at least 2D");
      }
      if (shape.back() != last_dim)
      {
        THROW_CAIFE(std::string(who) + ": last dim must match the adapter");
      }
      uint32_t n = 1;
      for (size_t i = 0; i + 1 < shape.size(); ++i)
      {
        n *= shape[i];
      }
      return n;
    }

    void UploadFp32(CAIF_DeviceTensor &dst, const std::vector<float> &host)
    {
      constexpr Dtype_e sd = Base_t::StorageDtype();
      if (sd == Dtype_e::Float32)
      {
        dst.CopyFromHostRaw(host.data(), host.size() * 4);
        return;
      }
      // 16-bit storage: upload fp32 to a scratch tensor and let the device cast round it (nearest even)
      CAIF_DeviceTensor tmp = CAIF_DeviceTensor::Uninitialized({static_cast<uint32_t>(host.size())}, Stream());
      tmp.CopyFromHostRaw(host.data(), host.size() * 4);
      CAIF_CheckCaifq(caifq_cast(tmp.DeviceDataRaw(), CAIFQ_F32, dst.DeviceDataRaw(), static_cast<int32_t>(sd),
                                 static_cast<int64_t>(host.size()), Stream().Handle()),
                      "LoRAAdapter: cast of the initial A");
      CAIF_CheckCuda(cudaStreamSynchronize(Stream().Handle()), "LoRAAdapter: init sync");
    }

    CAIF_DeviceLoRAAdapterConfig _config;
    std::unique_ptr<CAIF_DeviceLayer> _base_layer;
    CAIF_DeviceFrozenLinearBase *_frozen = nullptr;
    CAIF_DeviceTensor _lora_a;
    CAIF_DeviceTensor _lora_b;
    CAIF_DeviceTensor _grad_lora_a;
    CAIF_DeviceTensor _grad_lora_b;
    CAIF_DeviceTensor _cached_input;
    CAIF_DeviceTensor _cached_lora_hidden;
};

// ------------------------------------------------------------------ frozen MoE expert
class CAIF_DeviceMoEFrozenExpertConfig
{
  public:
    CAIF_DeviceMoEFrozenExpertConfig(uint32_t input_dim, uint32_t hidden_dim, bool use_gated)
        : _input_dim(input_dim), _hidden_dim(hidden_dim), _use_gated(use_gated)
    {
    }
    uint32_t InputDim() const { return _input_dim; }
    uint32_t HiddenDim() const { return _hidden_dim; }
    bool UseGated() const { return _use_gated; }

  private:
    uint32_t _input_dim;
    uint32_t _hidden_dim;
    bool _use_gated;
};

// down( silu(gate(x)) * up(x) ) over three frozen linears: src/caif_device_moe_frozen_expert.cpp:91-332.
// Only the gated (SwiGLU) form is built here.
template <typename ComputeT = float, typename StorageT = float>
class CAIF_DeviceMoEFrozenExpert : public CAIF_DeviceLayerTyped<ComputeT, StorageT>
{
  public:
    typedef CAIF_DeviceLayerTyped<ComputeT, StorageT> Base_t;
    using Base_t::Stream;
    using Dtype_e = CAIF_DataType::CAIF_DataType_e;

    struct FrozenSubLayers_t
    {
      std::unique_ptr<CAIF_DeviceFrozenLinearBase> gate;
      std::unique_ptr<CAIF_DeviceFrozenLinearBase> up;
      std::unique_ptr<CAIF_DeviceFrozenLinearBase> down;
    };

    CAIF_DeviceMoEFrozenExpert(const CAIF_DeviceMoEFrozenExpertConfig &config, FrozenSubLayers_t sub,
                               CAIF_CudaStream &stream)
        : Base_t(stream), _config(config), _sub(std::move(sub))
    {
      if (!_sub.up || !_sub.down || (config.UseGated() && !_sub.gate))
      {
        THROW_CAIFE("MoEFrozenExpert: sub-layers must not be null");
      }
    }

    CAIF_DeviceTensor ForwardImpl(const CAIF_DeviceTensor &input, CAIF_RunContext &ctx) override
    {
      const auto &shape = input.Shape();
      if (shape.size() != 2 || shape[1] != _config.InputDim())
      {
        THROW_CAIFE("MoEFrozenExpert::Forward: expected [N, input_dim]");
      }
      CAIF_DeviceTensor output = CAIF_DeviceTensor::Uninitialized({shape[0], _config.InputDim()}, Stream(),
                                                                  Base_t::StorageDtype());
      ForwardInto(input, output, ctx);
      return output;
    }

    // writes straight into `output_view` (a slice of the packed per-expert buffer):
    // include/caif/caif_device_moe_expert_base.h:75-86
    void ForwardInto(const CAIF_DeviceTensor &input, CAIF_DeviceTensor &output_view, CAIF_RunContext &ctx)
    {
      const uint32_t n = input.Shape()[0];
      constexpr Dtype_e sd = Base_t::StorageDtype();
      if (input.Dtype() != sd || output_view.Dtype() != sd)
      {
        THROW_CAIFE("MoEFrozenExpert::ForwardInto: tensors must be in the expert's storage dtype");
      }
      const bool gated = _config.UseGated();
      CAIF_DeviceTensor gate_out;
      if (gated)
      {
        gate_out = CAIF_DeviceTensor::Uninitialized({n, _config.HiddenDim()}, Stream(), sd);
      }
      CAIF_DeviceTensor up_out = CAIF_DeviceTensor::Uninitialized({n, _config.HiddenDim()}, Stream(), sd);
      CAIF_DeviceTensor hidden = CAIF_DeviceTensor::Uninitialized({n, _config.HiddenDim()}, Stream(), sd);
      caifq_weight g{};
      if (gated)
      {
        g = _sub.gate->AsCaifqWeight();
      }
      const caifq_weight u = _sub.up->AsCaifqWeight();
      const caifq_weight d = _sub.down->AsCaifqWeight();
      const int32_t offsets[2] = {0, static_cast<int32_t>(n)};
      CAIF_CheckCaifq(caifq_grouped_expert_fwd(gated ? &g : nullptr, &u, &d, 1, offsets, input.DeviceDataRaw(),
                                               output_view.DeviceDataRaw(), gate_out.DeviceDataRaw(),
                                               up_out.DeviceDataRaw(), hidden.DeviceDataRaw(),
                                               static_cast<int32_t>(sd), static_cast<int32_t>(Base_t::ComputeDtype()),
                                               Stream().Handle()),
                      "MoEFrozenExpert::Forward");
      if (ctx.Training())
      {
        _cached_gate_out = std::move(gate_out);
        _cached_up_out = std::move(up_out);
        _cached_rows = n;
      }
      // the temporaries are released in stream order when they go out of scope: no synchronisation
    }

    CAIF_DeviceTensor BackwardImpl(const CAIF_DeviceTensor &grad_output, CAIF_RunContext &) override
    {
      if (_cached_up_out.IsEmpty())
      {
        THROW_CAIFE("MoEFrozenExpert::Backward: must call Forward(training=true) first");
      }
      const bool gated = _config.UseGated();
      const uint32_t n = _cached_rows;
      constexpr Dtype_e sd = Base_t::StorageDtype();
      CAIF_DeviceTensor grad_input = CAIF_DeviceTensor::Uninitialized({n, _config.InputDim()}, Stream(), sd);
      CAIF_DeviceTensor ws = CAIF_DeviceTensor::Uninitialized({3u, n, _config.HiddenDim()}, Stream(), sd);
      caifq_weight g{};
      if (gated)
      {
        g = _sub.gate->AsCaifqWeight();
      }
      const caifq_weight u = _sub.up->AsCaifqWeight();
      const caifq_weight d = _sub.down->AsCaifqWeight();
      const int32_t offsets[2] = {0, static_cast<int32_t>(n)};
      CAIF_CheckCaifq(caifq_grouped_expert_bwd(gated ? &g : nullptr, &u, &d, 1, offsets, grad_output.DeviceDataRaw(),
                                               _cached_gate_out.DeviceDataRaw(), _cached_up_out.DeviceDataRaw(),
                                               grad_input.DeviceDataRaw(), ws.DeviceDataRaw(),
                                               static_cast<int32_t>(sd), static_cast<int32_t>(Base_t::ComputeDtype()),
                                               Stream().Handle()),
                      "MoEFrozenExpert::Backward");
      return grad_input;
    }

    CAIF_RunContext::Subsystem_e SubsystemTag() const override
    {
      return CAIF_RunContext::Subsystem_e::MoEFrozenExpert_e;
    }
    void ZeroGradients() override {}
    size_t ParameterTensorCount() const override { return 0; }
    CAIF_DeviceTensor &ParameterTensor(size_t) override { THROW_CAIFE("MoEFrozenExpert: no trainable parameters"); }
    CAIF_DeviceTensor &GradientTensor(size_t) override { THROW_CAIFE("MoEFrozenExpert: no trainable parameters"); }
    size_t TotalParameterCount() const override { return 0; }
    std::string Description() const override
    {
      return std::string("MoEFrozenExpert(") + std::to_string(_config.InputDim()) + "," +
             std::to_string(_config.HiddenDim()) + ")";
    }
    std::vector<std::string> ParameterNames(const std::string & = "") const override { return {}; }

    const CAIF_DeviceMoEFrozenExpertConfig &Config() const { return _config; }
    CAIF_DeviceFrozenLinearBase &Gate() { return *_sub.gate; }
    CAIF_DeviceFrozenLinearBase &Up() { return *_sub.up; }
    CAIF_DeviceFrozenLinearBase &Down() { return *_sub.down; }

  private:
    CAIF_DeviceMoEFrozenExpertConfig _config;
    FrozenSubLayers_t _sub;
    CAIF_DeviceTensor _cached_gate_out;
    CAIF_DeviceTensor _cached_up_out;
    uint32_t _cached_rows = 0;
};

}  // namespace instance
