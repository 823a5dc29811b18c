// SafeTensors files of quantized frozen weights: the on-disk side of the frozen-linear path.
//
// Mirrors the interface of the reference's CAIF_SafeTensorsFormat (include/caif/caif_safetensors_format.h:40-262,
// src/caif_safetensors_format.cpp) and CAIF_WeightMapper (include/caif/caif_weight_mapper.h,
// src/caif_weight_mapper.cpp) over this library's tensor type: same method names, same dtype vocabulary
// ("F32", "F16", "BF16", "I8", and the reference's own "I4" with two codes per byte, low nibble first, so a
// tensor of n elements occupies (n + 1) / 2 bytes), same file layout (8-byte little-endian header length, JSON
// header padded with spaces to a multiple of 8, tensors back to back in the order given, "__metadata__" last),
// same refusals (header or file too small / too large, offsets that do not match dtype x shape or run past the
// file, unknown dtype names, more than 4096 tensors).  Files written here load in the reference and the other
// way round.
//
// Built differently: a file is opened once (CAIF_SafeTensorsFile), its header parsed into an index by a small
// general JSON reader, and tensors are fetched on demand with pread into pinned staging and copied to the
// device on the caller's stream; the reference re-opens and re-parses the file for every tensor it loads.
// LoadFrozenLinear feeds a CAIF_DeviceFrozenLinearBase straight from a file: codes + scales as stored, or a
// float weight quantized on the device with the bit-exact quantizers when the layer stores int8 / int4.
#pragma once

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <sstream>
#include <string>
#include <utility>
#include <variant>
#include <vector>

#include "caif_host.hpp"

namespace instance
{

constexpr uint64_t g_caif_safetensors_max_file_size = 2ULL << 40;
constexpr size_t g_caif_safetensors_max_tensors = 4096;
constexpr size_t g_caif_safetensors_max_header_size = 100 * 1024 * 1024;

// ----------------------------------------------------------------------- JSON
// Just enough JSON for a SafeTensors header and a shard index: objects, arrays, strings with the usual
// escapes, non-negative integers (other numbers are kept as text), true / false / null.
struct CAIF_JsonValue
{
    using Object = std::vector<std::pair<std::string, CAIF_JsonValue>>;   // insertion order kept
    using Array = std::vector<CAIF_JsonValue>;
    std::variant<std::monostate, bool, uint64_t, std::string, std::shared_ptr<Object>, std::shared_ptr<Array>> v;
    bool number_as_text = false;

    const Object *AsObject() const
    {
      auto p = std::get_if<std::shared_ptr<Object>>(&v);
      return p ? p->get() : nullptr;
    }
    const Array *AsArray() const
    {
      auto p = std::get_if<std::shared_ptr<Array>>(&v);
      return p ? p->get() : nullptr;
    }
    const std::string *AsString() const { return number_as_text ? nullptr : std::get_if<std::string>(&v); }
    const uint64_t *AsUnsigned() const { return std::get_if<uint64_t>(&v); }
    const CAIF_JsonValue *Find(const std::string &key) const
    {
      if (const Object *o = AsObject())
      {
        for (const auto &kv : *o)
        {
          if (kv.first == key)
          {
            return &kv.second;
          }
        }
      }
      return nullptr;
    }
};

class CAIF_JsonReader
{
  public:
    explicit CAIF_JsonReader(const std::string &text) : _s(text), _i(0) {}

    CAIF_JsonValue Parse()
    {
      CAIF_JsonValue v = Value(0);
      Blank();
      if (_i != _s.size())
      {
        Fail("trailing characters after the JSON value");
      }
      return v;
    }

  private:
    [[noreturn]] void Fail(const char *what) const
    {
      THROW_CAIFE(std::string("SafeTensors: malformed JSON header: ") + what + " at byte " + std::to_string(_i));
    }
    void Blank()
    {
      while (_i < _s.size() && (_s[_i] == ' ' || _s[_i] == '\n' || _s[_i] == '\r' || _s[_i] == '\t'))
      {
        ++_i;
      }
    }
    char Peek()
    {
      Blank();
      if (_i >= _s.size())
      {
        Fail("unexpected end");
      }
      return _s[_i];
    }
    void Expect(char c)
    {
      if (Peek() != c)
      {
        Fail("unexpected character");
      }
      ++_i;
    }
    static void AppendUtf8(std::string &out, uint32_t cp)
    {
      if (cp < 0x80)
      {
        out += static_cast<char>(cp);
      }
      else if (cp < 0x800)
      {
        out += static_cast<char>(0xC0 | (cp >> 6));
        out += static_cast<char>(0x80 | (cp & 0x3F));
      }
      else if (cp < 0x10000)
      {
        out += static_cast<char>(0xE0 | (cp >> 12));
        out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
        out += static_cast<char>(0x80 | (cp & 0x3F));
      }
      else
      {
        out += static_cast<char>(0xF0 | (cp >> 18));
        out += static_cast<char>(0x80 | ((cp >> 12) & 0x3F));
        out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F));
        out += static_cast<char>(0x80 | (cp & 0x3F));
      }
    }
    uint32_t Hex4()
    {
      if (_i + 4 > _s.size())
      {
        Fail("short \\u escape");
      }
      uint32_t v = 0;
      for (int k = 0; k < 4; ++k)
      {
        const char c = _s[_i++];
        v <<= 4;
        if (c >= '0' && c <= '9')
        {
          v |= static_cast<uint32_t>(c - '0');
        }
        else if (c >= 'a' && c <= 'f')
        {
          v |= static_cast<uint32_t>(c - 'a' + 10);
        }
        else if (c >= 'A' && c <= 'F')
        {
          v |= static_cast<uint32_t>(c - 'A' + 10);
        }
        else
        {
          Fail("bad \\u escape");
        }
      }
      return v;
    }
    std::string String()
    {
      Expect('"');
      std::string out;
      for (;;)
      {
        if (_i >= _s.size())
        {
          Fail("unterminated string");
        }
        const char c = _s[_i++];
        if (c == '"')
        {
          return out;
        }
        if (c != '\\')
        {
          out += c;
          continue;
        }
        if (_i >= _s.size())
        {
          Fail("unterminated escape");
        }
        const char e = _s[_i++];
        switch (e)
        {
          case '"': out += '"'; break;
          case '\\': out += '\\'; break;
          case '/': out += '/'; break;
          case 'b': out += '\b'; break;
          case 'f': out += '\f'; break;
          case 'n': out += '\n'; break;
          case 'r': out += '\r'; break;
          case 't': out += '\t'; break;
          case 'u':
          {
            uint32_t cp = Hex4();
            if (cp >= 0xD800 && cp < 0xDC00 && _i + 1 < _s.size() && _s[_i] == '\\' && _s[_i + 1] == 'u')
            {
              _i += 2;
              const uint32_t lo = Hex4();
              cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
            }
            AppendUtf8(out, cp);
            break;
          }
          default: Fail("unknown escape");
        }
      }
    }
    CAIF_JsonValue Value(int depth)
    {
      if (depth > 32)
      {
        Fail("nesting too deep");
      }
      CAIF_JsonValue out;
      const char c = Peek();
      if (c == '{')
      {
        ++_i;
        auto obj = std::make_shared<CAIF_JsonValue::Object>();
        if (Peek() == '}')
        {
          ++_i;
        }
        else
        {
          for (;;)
          {
            Blank();
            std::string key = String();
            Expect(':');
            obj->emplace_back(std::move(key), Value(depth + 1));
            if (Peek() == ',')
            {
              ++_i;
              continue;
            }
            Expect('}');
            break;
          }
        }
        out.v = std::move(obj);
      }
      else if (c == '[')
      {
        ++_i;
        auto arr = std::make_shared<CAIF_JsonValue::Array>();
        if (Peek() == ']')
        {
          ++_i;
        }
        else
        {
          for (;;)
          {
            arr->push_back(Value(depth + 1));
            if (Peek() == ',')
            {
              ++_i;
              continue;
            }
            Expect(']');
            break;
          }
        }
        out.v = std::move(arr);
      }
      else if (c == '"')
      {
        out.v = String();
      }
      else if (_s.compare(_i, 4, "true") == 0)
      {
        _i += 4;
        out.v = true;
      }
      else if (_s.compare(_i, 5, "false") == 0)
      {
        _i += 5;
        out.v = false;
      }
      else if (_s.compare(_i, 4, "null") == 0)
      {
        _i += 4;
      }
      else
      {
        const size_t start = _i;
        bool integer = true;
        while (_i < _s.size() && (std::strchr("+-.eE", _s[_i]) != nullptr || (_s[_i] >= '0' && _s[_i] <= '9')))
        {
          integer = integer && _s[_i] >= '0' && _s[_i] <= '9';
          ++_i;
        }
        if (_i == start)
        {
          Fail("unexpected character");
        }
        if (integer && _i - start <= 19)
        {
          out.v = static_cast<uint64_t>(std::stoull(_s.substr(start, _i - start)));
        }
        else
        {
          out.v = _s.substr(start, _i - start);   // kept as text; never a shape or an offset
          out.number_as_text = true;
        }
      }
      return out;
    }

    const std::string &_s;
    size_t _i;
};

// ------------------------------------------------------------------ dtype names
struct CAIF_SafeTensorsDtype
{
    const char *name;
    int bits;          // per element
    int caif_dtype;    // CAIF_DataType_e value, -1 when this library has no tensor type for it
};

inline const std::vector<CAIF_SafeTensorsDtype> &CAIF_SafeTensorsDtypes()
{
  using E = CAIF_DataType::CAIF_DataType_e;
  static const std::vector<CAIF_SafeTensorsDtype> table = {
      {"F32", 32, static_cast<int>(E::Float32)}, {"F64", 64, static_cast<int>(E::Float64)},
      {"F16", 16, static_cast<int>(E::Float16)}, {"BF16", 16, static_cast<int>(E::BFloat16)},
      {"I4", 4, static_cast<int>(E::Int4)},      {"I8", 8, static_cast<int>(E::Int8)},
      {"I16", 16, -1},                           {"I32", 32, -1},
      {"I64", 64, -1},                           {"U8", 8, -1},
      {"U16", 16, -1},                           {"U32", 32, -1},
      {"U64", 64, -1},                           {"BOOL", 8, -1}};
  return table;
}

// ------------------------------------------------------------------- one file
class CAIF_SafeTensorsFile
{
  public:
    struct SafeTensorInfo_t
    {
        std::string dtype;
        std::vector<uint32_t> shape;
        uint64_t data_offset_start = 0;
        uint64_t data_offset_end = 0;
    };
    using InfoMap_t = std::map<std::string, SafeTensorInfo_t>;

    explicit CAIF_SafeTensorsFile(const std::string &path) : _path(path)
    {
      _fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
      if (_fd < 0)
      {
        THROW_CAIFE("SafeTensors: cannot open file: " + path);
      }
      try
      {
        ReadIndex();
      }
      catch (...)
      {
        ::close(_fd);
        throw;
      }
    }
    CAIF_SafeTensorsFile(const CAIF_SafeTensorsFile &) = delete;
    CAIF_SafeTensorsFile &operator=(const CAIF_SafeTensorsFile &) = delete;
    ~CAIF_SafeTensorsFile()
    {
      if (_fd >= 0)
      {
        ::close(_fd);
      }
    }

    const std::string &Path() const { return _path; }
    uint64_t DataStart() const { return _data_start; }
    const InfoMap_t &TensorInfos() const { return _infos; }
    const std::vector<std::string> &NamesInFileOrder() const { return _order; }
    const std::map<std::string, std::string> &Metadata() const { return _metadata; }

    const SafeTensorInfo_t &Info(const std::string &name) const
    {
      const auto it = _infos.find(name);
      if (it == _infos.end())
      {
        THROW_CAIFE("SafeTensors: tensor '" + name + "' not found in " + _path);
      }
      return it->second;
    }

    static const CAIF_SafeTensorsDtype &DtypeEntry(const std::string &name)
    {
      for (const auto &d : CAIF_SafeTensorsDtypes())
      {
        if (name == d.name)
        {
          return d;
        }
      }
      THROW_CAIFE("CAIF_SafeTensorsFormat::DtypeFromSafeTensorsName: unrecognised name");
    }

    // Bytes the tensor must occupy: dtype x shape, validated against its offsets and the file.
    uint64_t CheckedBytes(const SafeTensorInfo_t &info) const
    {
      const CAIF_SafeTensorsDtype &d = DtypeEntry(info.dtype);
      uint64_t elements = 1;
      for (uint32_t dim : info.shape)
      {
        elements *= dim;
      }
      const uint64_t expected = (elements * static_cast<uint64_t>(d.bits) + 7) / 8;
      if (info.data_offset_start > info.data_offset_end)
      {
        THROW_CAIFE("SafeTensors: data_offset_start exceeds data_offset_end");
      }
      if (info.data_offset_end - info.data_offset_start != expected)
      {
        THROW_CAIFE("SafeTensors: data size mismatch");
      }
      if (_data_start > _file_size || info.data_offset_end > _file_size - _data_start)
      {
        THROW_CAIFE("SafeTensors: tensor data extends past end of file");
      }
      return expected;
    }

    // The tensor's bytes into host memory.
    void ReadRaw(const std::string &name, void *dst, size_t capacity) const
    {
      const SafeTensorInfo_t &info = Info(name);
      const uint64_t bytes = CheckedBytes(info);
      if (bytes > capacity)
      {
        THROW_CAIFE("SafeTensors: destination too small for tensor '" + name + "'");
      }
      uint64_t done = 0;
      while (done < bytes)
      {
        const ssize_t got = ::pread(_fd, static_cast<char *>(dst) + done, bytes - done,
                                    static_cast<off_t>(_data_start + info.data_offset_start + done));
        if (got <= 0)
        {
          THROW_CAIFE("SafeTensors: short read loading tensor data");
        }
        done += static_cast<uint64_t>(got);
      }
    }

    // The tensor on the device with its native dtype, through pinned staging on `stream`.
    CAIF_DeviceTensor Load(const std::string &name, const CAIF_CudaStream &stream) const
    {
      const SafeTensorInfo_t &info = Info(name);
      const CAIF_SafeTensorsDtype &d = DtypeEntry(info.dtype);
      if (d.caif_dtype < 0)
      {
        THROW_CAIFE("SafeTensors: dtype " + info.dtype + " of tensor '" + name + "' has no device tensor type");
      }
      const uint64_t bytes = CheckedBytes(info);
      CAIF_DeviceTensor t = CAIF_DeviceTensor::Uninitialized(
          info.shape, stream, static_cast<CAIF_DataType::CAIF_DataType_e>(d.caif_dtype));
      if (bytes == 0)
      {
        return t;
      }
      void *pinned = nullptr;
      CAIF_CheckCuda(cudaMallocHost(&pinned, bytes), "SafeTensors: pinned staging");
      try
      {
        ReadRaw(name, pinned, bytes);
        t.CopyFromHostRaw(pinned, bytes);   // synchronizes the stream: the staging can go
      }
      catch (...)
      {
        cudaFreeHost(pinned);
        throw;
      }
      cudaFreeHost(pinned);
      return t;
    }

  private:
    void ReadIndex()
    {
      struct stat st;
      if (::fstat(_fd, &st) != 0)
      {
        THROW_CAIFE("SafeTensors: cannot determine file size");
      }
      _file_size = static_cast<uint64_t>(st.st_size);
      if (_file_size < 8)
      {
        THROW_CAIFE("SafeTensors: file too small");
      }
      if (_file_size > g_caif_safetensors_max_file_size)
      {
        THROW_CAIFE("SafeTensors: file too large");
      }
      uint64_t header_size = 0;
      if (::pread(_fd, &header_size, 8, 0) != 8)
      {
        THROW_CAIFE("SafeTensors: file too small");
      }
      if (header_size > g_caif_safetensors_max_header_size)
      {
        THROW_CAIFE("SafeTensors: header too large");
      }
      if (8 + header_size > _file_size)
      {
        THROW_CAIFE("SafeTensors: invalid header size");
      }
      std::string json(static_cast<size_t>(header_size), '\0');
      uint64_t done = 0;
      while (done < header_size)
      {
        const ssize_t got = ::pread(_fd, json.data() + done, header_size - done, static_cast<off_t>(8 + done));
        if (got <= 0)
        {
          THROW_CAIFE("SafeTensors: invalid header size");
        }
        done += static_cast<uint64_t>(got);
      }
      _data_start = 8 + header_size;
      const CAIF_JsonValue root = CAIF_JsonReader(json).Parse();
      const CAIF_JsonValue::Object *entries = root.AsObject();
      if (entries == nullptr)
      {
        THROW_CAIFE("SafeTensors: header is not a JSON object");
      }
      for (const auto &kv : *entries)
      {
        if (kv.first == "__metadata__")
        {
          if (const CAIF_JsonValue::Object *meta = kv.second.AsObject())
          {
            for (const auto &m : *meta)
            {
              if (const std::string *text = m.second.AsString())
              {
                _metadata[m.first] = *text;
              }
            }
          }
          continue;
        }
        SafeTensorInfo_t info;
        const CAIF_JsonValue *dtype = kv.second.Find("dtype");
        const CAIF_JsonValue *shape = kv.second.Find("shape");
        const CAIF_JsonValue *offsets = kv.second.Find("data_offsets");
        if (dtype == nullptr || dtype->AsString() == nullptr || shape == nullptr || shape->AsArray() == nullptr ||
            offsets == nullptr || offsets->AsArray() == nullptr || offsets->AsArray()->size() != 2)
        {
          THROW_CAIFE("SafeTensors: tensor '" + kv.first + "' needs dtype, shape and two data_offsets");
        }
        info.dtype = *dtype->AsString();
        for (const CAIF_JsonValue &dim : *shape->AsArray())
        {
          const uint64_t *n = dim.AsUnsigned();
          if (n == nullptr || *n > 0xFFFFFFFFull)
          {
            THROW_CAIFE("SafeTensors: tensor '" + kv.first + "' has a bad shape entry");
          }
          info.shape.push_back(static_cast<uint32_t>(*n));
        }
        const uint64_t *b = (*offsets->AsArray())[0].AsUnsigned();
        const uint64_t *e = (*offsets->AsArray())[1].AsUnsigned();
        if (b == nullptr || e == nullptr)
        {
          THROW_CAIFE("SafeTensors: tensor '" + kv.first + "' has bad data_offsets");
        }
        info.data_offset_start = *b;
        info.data_offset_end = *e;
        if (_infos.emplace(kv.first, std::move(info)).second)
        {
          _order.push_back(kv.first);
        }
      }
      if (_infos.size() > g_caif_safetensors_max_tensors)
      {
        THROW_CAIFE("SafeTensors: too many tensors");
      }
    }

    std::string _path;
    int _fd = -1;
    uint64_t _file_size = 0;
    uint64_t _data_start = 0;
    InfoMap_t _infos;
    std::vector<std::string> _order;
    std::map<std::string, std::string> _metadata;
};

// --------------------------------------------------------------- the format
class CAIF_SafeTensorsFormat
{
  public:
    using SafeTensorInfo_t = CAIF_SafeTensorsFile::SafeTensorInfo_t;
    using Dtype_e = CAIF_DataType::CAIF_DataType_e;

    // A tensor to be written: device tensors are downloaded, host blobs are written as they are.
    struct HostBlob_t
    {
        std::string dtype;              // SafeTensors name
        std::vector<uint32_t> shape;
        const void *data = nullptr;     // (elements x bits + 7) / 8 bytes
    };

    static const std::string &DtypeToSafeTensorsName(Dtype_e dt)
    {
      static const std::map<Dtype_e, std::string> names = []()
      {
        std::map<Dtype_e, std::string> m;
        for (const auto &d : CAIF_SafeTensorsDtypes())
        {
          if (d.caif_dtype >= 0)
          {
            m[static_cast<Dtype_e>(d.caif_dtype)] = d.name;
          }
        }
        return m;
      }();
      const auto it = names.find(dt);
      if (it == names.end())
      {
        THROW_CAIFE("CAIF_SafeTensorsFormat::DtypeToSafeTensorsName: unsupported dtype");
      }
      return it->second;
    }

    static Dtype_e DtypeFromSafeTensorsName(const std::string &name)
    {
      const CAIF_SafeTensorsDtype &d = CAIF_SafeTensorsFile::DtypeEntry(name);
      if (d.caif_dtype < 0)
      {
        THROW_CAIFE("CAIF_SafeTensorsFormat::DtypeFromSafeTensorsName: unrecognised name");
      }
      return static_cast<Dtype_e>(d.caif_dtype);
    }

    std::string Extension() const { return ".safetensors"; }
    std::string FormatName() const { return "SafeTensors"; }

    void Save(const std::string &path, const std::vector<std::pair<std::string, const CAIF_DeviceTensor *>> &tensors,
              const std::map<std::string, std::string> &metadata) const
    {
      std::vector<std::vector<char>> staged;
      std::vector<std::pair<std::string, HostBlob_t>> blobs;
      staged.reserve(tensors.size());
      for (const auto &kv : tensors)
      {
        if (kv.second == nullptr)
        {
          continue;
        }
        staged.emplace_back(kv.second->SizeBytes());
        if (!staged.back().empty())
        {
          kv.second->CopyToHostRaw(staged.back().data());
        }
        HostBlob_t blob;
        blob.dtype = DtypeToSafeTensorsName(kv.second->Dtype());
        blob.shape = kv.second->Shape();
        blob.data = staged.back().data();
        blobs.emplace_back(kv.first, blob);
      }
      SaveHost(path, blobs, metadata);
    }

    void SaveHost(const std::string &path, const std::vector<std::pair<std::string, HostBlob_t>> &tensors,
                  const std::map<std::string, std::string> &metadata) const
    {
      if (tensors.size() > g_caif_safetensors_max_tensors)
      {
        THROW_CAIFE("SafeTensors: too many tensors");
      }
      std::ostringstream json;
      std::vector<uint64_t> sizes;
      uint64_t cursor = 0;
      const char *sep = "";
      json << "{";
      for (const auto &kv : tensors)
      {
        const CAIF_SafeTensorsDtype &d = CAIF_SafeTensorsFile::DtypeEntry(kv.second.dtype);
        uint64_t elements = 1;
        json << sep << "\"" << EscapeJsonString(kv.first) << "\":{\"dtype\":\"" << d.name << "\",\"shape\":[";
        for (size_t i = 0; i < kv.second.shape.size(); ++i)
        {
          elements *= kv.second.shape[i];
          json << (i ? "," : "") << kv.second.shape[i];
        }
        const uint64_t bytes = (elements * static_cast<uint64_t>(d.bits) + 7) / 8;
        json << "],\"data_offsets\":[" << cursor << "," << cursor + bytes << "]}";
        cursor += bytes;
        sizes.push_back(bytes);
        sep = ",";
      }
      if (!metadata.empty())
      {
        json << sep << "\"__metadata__\":{";
        const char *msep = "";
        for (const auto &kv : metadata)
        {
          json << msep << "\"" << EscapeJsonString(kv.first) << "\":\"" << EscapeJsonString(kv.second) << "\"";
          msep = ",";
        }
        json << "}";
      }
      json << "}";
      std::string header = json.str();
      header.append((8 - header.size() % 8) % 8, ' ');
      if (header.size() > g_caif_safetensors_max_header_size)
      {
        THROW_CAIFE("SafeTensors: header too large");
      }
      const int fd = ::open(path.c_str(), O_WRONLY | O_CREAT | O_TRUNC | O_CLOEXEC, 0644);
      if (fd < 0)
      {
        THROW_CAIFE("SafeTensors: cannot open file for writing: " + path);
      }
      const uint64_t header_size = header.size();
      bool ok = WriteAll(fd, &header_size, 8) && WriteAll(fd, header.data(), header.size());
      for (size_t i = 0; ok && i < tensors.size(); ++i)
      {
        ok = sizes[i] == 0 || WriteAll(fd, tensors[i].second.data, sizes[i]);
      }
      ok = (::close(fd) == 0) && ok;
      if (!ok)
      {
        THROW_CAIFE("SafeTensors: write failed: " + path);
      }
    }

    std::map<std::string, CAIF_DeviceTensor> Load(const std::string &path, CAIF_CudaStream &stream) const
    {
      CAIF_SafeTensorsFile file(path);
      std::map<std::string, CAIF_DeviceTensor> out;
      for (const auto &kv : file.TensorInfos())
      {
        out.emplace(kv.first, file.Load(kv.first, stream));
      }
      return out;
    }

    std::map<std::string, std::string> Metadata(const std::string &path) const
    {
      return CAIF_SafeTensorsFile(path).Metadata();
    }

    std::map<std::string, SafeTensorInfo_t> TensorInfos(const std::string &path) const
    {
      return CAIF_SafeTensorsFile(path).TensorInfos();
    }

    // A checkpoint directory: model.safetensors.index.json with a "weight_map" of tensor name -> shard file,
    // or a single model.safetensors.  Shards are opened on first use and stay open with the handle.
    class ShardedHandle_t
    {
      public:
        const std::string &Directory() const { return _directory; }
        const std::map<std::string, std::string> &WeightMap() const { return _weight_map; }

        const CAIF_SafeTensorsFile &ShardOf(const std::string &tensor_name) const
        {
          const auto it = _weight_map.find(tensor_name);
          if (it == _weight_map.end())
          {
            THROW_CAIFE("SafeTensors: tensor '" + tensor_name + "' not found in weight map of " + _directory);
          }
          auto &slot = _shards[it->second];
          if (!slot)
          {
            slot = std::make_unique<CAIF_SafeTensorsFile>(_directory + "/" + it->second);
          }
          return *slot;
        }

      private:
        friend class CAIF_SafeTensorsFormat;
        std::string _directory;
        std::map<std::string, std::string> _weight_map;
        mutable std::map<std::string, std::unique_ptr<CAIF_SafeTensorsFile>> _shards;
    };

    ShardedHandle_t OpenShardedHandle(const std::string &directory) const
    {
      ShardedHandle_t handle;
      handle._directory = directory;
      const std::string index_path = directory + "/model.safetensors.index.json";
      const std::string single = "model.safetensors";
      if (::access(index_path.c_str(), R_OK) == 0)
      {
        handle._weight_map = ParseShardIndex(index_path);
        if (handle._weight_map.empty())
        {
          THROW_CAIFE("SafeTensors: empty weight map in index file");
        }
        return handle;
      }
      if (::access((directory + "/" + single).c_str(), R_OK) != 0)
      {
        THROW_CAIFE("SafeTensors: no index file and no model.safetensors in " + directory);
      }
      auto file = std::make_unique<CAIF_SafeTensorsFile>(directory + "/" + single);
      for (const auto &kv : file->TensorInfos())
      {
        handle._weight_map[kv.first] = single;
      }
      if (handle._weight_map.empty())
      {
        THROW_CAIFE("SafeTensors: single-shard model.safetensors has no tensors in " + directory);
      }
      handle._shards[single] = std::move(file);
      return handle;
    }

    CAIF_DeviceTensor LoadFromHandle(const ShardedHandle_t &handle, const std::string &tensor_name,
                                     CAIF_CudaStream &stream) const
    {
      return handle.ShardOf(tensor_name).Load(tensor_name, stream);
    }

    CAIF_DeviceTensor LoadTensorByName(const std::string &directory, const std::string &tensor_name,
                                       CAIF_CudaStream &stream) const
    {
      return LoadFromHandle(OpenShardedHandle(directory), tensor_name, stream);
    }

    std::map<std::string, CAIF_DeviceTensor> LoadSharded(const std::string &directory, CAIF_CudaStream &stream) const
    {
      const ShardedHandle_t handle = OpenShardedHandle(directory);
      std::map<std::string, CAIF_DeviceTensor> out;
      for (const auto &kv : handle.WeightMap())
      {
        out.emplace(kv.first, LoadFromHandle(handle, kv.first, stream));
      }
      return out;
    }

    static std::map<std::string, std::string> ParseShardIndex(const std::string &index_path)
    {
      const int fd = ::open(index_path.c_str(), O_RDONLY | O_CLOEXEC);
      if (fd < 0)
      {
        THROW_CAIFE("SafeTensors: cannot open index file: " + index_path);
      }
      std::string text;
      char chunk[1 << 16];
      ssize_t got = 0;
      while ((got = ::read(fd, chunk, sizeof(chunk))) > 0)
      {
        text.append(chunk, static_cast<size_t>(got));
      }
      ::close(fd);
      const CAIF_JsonValue root = CAIF_JsonReader(text).Parse();
      std::map<std::string, std::string> out;
      if (const CAIF_JsonValue *wm = root.Find("weight_map"))
      {
        if (const CAIF_JsonValue::Object *o = wm->AsObject())
        {
          for (const auto &kv : *o)
          {
            if (const std::string *file = kv.second.AsString())
            {
              out[kv.first] = *file;
            }
          }
        }
      }
      return out;
    }

    static std::string EscapeJsonString(const std::string &s)
    {
      std::string out;
      out.reserve(s.size() + 8);
      for (const char c : s)
      {
        switch (c)
        {
          case '"': out += "\\\""; break;
          case '\\': out += "\\\\"; break;
          case '\n': out += "\\n"; break;
          case '\r': out += "\\r"; break;
          case '\t': out += "\\t"; break;
          default: out += c;
        }
      }
      return out;
    }

  private:
    static bool WriteAll(int fd, const void *data, uint64_t bytes)
    {
      uint64_t done = 0;
      while (done < bytes)
      {
        const ssize_t put = ::write(fd, static_cast<const char *>(data) + done, bytes - done);
        if (put <= 0)
        {
          return false;
        }
        done += static_cast<uint64_t>(put);
      }
      return true;
    }
};

// ------------------------------------------------------------ name mapping
// Hugging Face <-> CAIF tensor names: exact aliases win, otherwise the rule with the longest matching
// prefix rewrites the prefix; no match gives "".
class CAIF_WeightMapper
{
  public:
    void AddPrefixRule(const std::string &hf_prefix, const std::string &aif_prefix)
    {
      _rules.emplace_back(hf_prefix, aif_prefix);
    }
    void AddAlias(const std::string &hf_name, const std::string &aif_name)
    {
      _hf_to_aif[hf_name] = aif_name;
      _aif_to_hf[aif_name] = hf_name;
    }
    std::string HfToAif(const std::string &hf_name) const { return Translate(hf_name, _hf_to_aif, true); }
    std::string AifToHf(const std::string &aif_name) const { return Translate(aif_name, _aif_to_hf, false); }

    std::vector<std::pair<std::string, std::string>> RequiredHfNames(const std::vector<std::string> &aif_names) const
    {
      std::vector<std::pair<std::string, std::string>> out;
      for (const std::string &aif : aif_names)
      {
        std::string hf = AifToHf(aif);
        if (!hf.empty())
        {
          out.emplace_back(std::move(hf), aif);
        }
      }
      return out;
    }
    std::vector<std::string> MissingNames(const std::vector<std::string> &aif_names,
                                          const std::set<std::string> &available_hf_names) const
    {
      std::vector<std::string> out;
      for (const std::string &aif : aif_names)
      {
        const std::string hf = AifToHf(aif);
        if (hf.empty() || available_hf_names.count(hf) == 0)
        {
          out.push_back(aif);
        }
      }
      return out;
    }
    std::vector<std::string> UnmappedHfNames(const std::set<std::string> &available_hf_names) const
    {
      std::vector<std::string> out;
      std::copy_if(available_hf_names.begin(), available_hf_names.end(), std::back_inserter(out),
                   [this](const std::string &hf) { return HfToAif(hf).empty(); });
      return out;
    }
    size_t PrefixRuleCount() const { return _rules.size(); }
    size_t AliasCount() const { return _hf_to_aif.size(); }

  private:
    std::string Translate(const std::string &name, const std::map<std::string, std::string> &aliases,
                          bool from_hf) const
    {
      const auto alias = aliases.find(name);
      if (alias != aliases.end())
      {
        return alias->second;
      }
      const std::pair<std::string, std::string> *best = nullptr;
      for (const auto &rule : _rules)
      {
        const std::string &from = from_hf ? rule.first : rule.second;
        const bool longer = best == nullptr || from.size() > (from_hf ? best->first : best->second).size();
        if (longer && name.compare(0, from.size(), from) == 0)
        {
          best = &rule;
        }
      }
      if (best == nullptr)
      {
        return "";
      }
      const std::string &from = from_hf ? best->first : best->second;
      const std::string &to = from_hf ? best->second : best->first;
      return to + name.substr(from.size());
    }

    std::vector<std::pair<std::string, std::string>> _rules;   // (hf prefix, aif prefix)
    std::map<std::string, std::string> _hf_to_aif;
    std::map<std::string, std::string> _aif_to_hf;
};

// -------------------------------------------------- file -> frozen linear layer
// Feeds a frozen linear from a checkpoint.  The weight tensor must hold input_dim x output_dim elements.
//  * stored dtype == the layer's storage dtype: the bytes go to LoadFromTensor as they are; an int8 / int4
//    layer then takes its scales from `scales_name` (F32 for int8: one value, or one per output row; F16 for
//    int4: one per group) through LoadScalesFromHost.
//  * a float tensor (F32 / F16 / BF16) for an int8 / int4 layer: quantized on the device at load time with
//    caifq_quantize_int8_per_tensor / caifq_quantize_int4_per_group (the reference's arithmetic bit for bit,
//    src/caif_cuda_kernels_quant.cu), codes to LoadFromTensor and the device-computed scales to the layer.
//  * a float tensor for a float layer of another dtype: converted with caifq_cast.
inline void LoadFrozenLinear(CAIF_DeviceFrozenLinearBase &layer, const CAIF_SafeTensorsFile &file,
                             const std::string &weight_name, const std::string &scales_name,
                             CAIF_CudaStream &stream)
{
  using E = CAIF_DataType::CAIF_DataType_e;
  const auto code_of = [](E d) -> int
  {
    switch (d)
    {
      case E::Float32: return CAIFQ_F32;
      case E::Float16: return CAIFQ_F16;
      case E::BFloat16: return CAIFQ_BF16;
      case E::Int8: return CAIFQ_I8;
      case E::Int4: return CAIFQ_I4;
      default: break;
    }
    THROW_CAIFE("LoadFrozenLinear: dtype has no kernel code");
  };
  const E want = layer.WeightStorageDtype();
  const uint32_t group_size = layer.QuantGroupSize();
  CAIF_DeviceTensor stored = file.Load(weight_name, stream);
  const size_t elements = stored.NumElements();
  const bool stored_float = stored.Dtype() == E::Float32 || stored.Dtype() == E::Float16 || stored.Dtype() == E::BFloat16;
  if (stored.Dtype() == want)
  {
    layer.LoadFromTensor(std::move(stored));
    if (layer.NeedsScales())
    {
      if (scales_name.empty())
      {
        THROW_CAIFE("LoadFrozenLinear: quantized tensor '" + weight_name + "' needs a scales tensor");
      }
      const auto &info = file.Info(scales_name);
      std::vector<char> host(file.CheckedBytes(info));
      file.ReadRaw(scales_name, host.data(), host.size());
      layer.LoadScalesFromHost(host.data(), host.size());
    }
    return;
  }
  if (!stored_float)
  {
    THROW_CAIFE("LoadFrozenLinear: tensor '" + weight_name + "' is " +
                CAIF_SafeTensorsFormat::DtypeToSafeTensorsName(stored.Dtype()) + ", the layer stores " +
                CAIF_DataType::Name(want));
  }
  // to fp32 first where the quantizers want it
  CAIF_DeviceTensor f32;
  const void *src_f32 = stored.DeviceDataRaw();
  if (stored.Dtype() != E::Float32 && (want == E::Int8 || want == E::Int4))
  {
    f32 = CAIF_DeviceTensor::Uninitialized(stored.Shape(), stream, E::Float32);
    CAIF_CheckCaifq(caifq_cast(stored.DeviceDataRaw(), code_of(stored.Dtype()), f32.DeviceDataRaw(), CAIFQ_F32,
                               static_cast<int64_t>(elements), stream.Handle()),
                    "LoadFrozenLinear: cast");
    src_f32 = f32.DeviceDataRaw();
  }
  if (want == E::Int8)
  {
    CAIF_DeviceTensor codes = CAIF_DeviceTensor::Uninitialized(stored.Shape(), stream, E::Int8);
    CAIF_DeviceTensor scale = CAIF_DeviceTensor::Uninitialized({1}, stream, E::Float32);
    CAIF_CheckCaifq(caifq_quantize_int8_per_tensor(static_cast<const float *>(src_f32),
                                                   static_cast<int8_t *>(codes.DeviceDataRaw()),
                                                   static_cast<float *>(scale.DeviceDataRaw()),
                                                   static_cast<int64_t>(elements), stream.Handle()),
                    "LoadFrozenLinear: quantize int8");
    float host_scale = 0.0f;
    scale.CopyToHostRaw(&host_scale);
    layer.LoadFromTensor(std::move(codes));
    layer.LoadScalesFromHost(&host_scale, sizeof(float));
    return;
  }
  if (want == E::Int4)
  {
    const size_t groups = (elements + group_size - 1) / group_size;
    CAIF_DeviceTensor codes = CAIF_DeviceTensor::Uninitialized(stored.Shape(), stream, E::Int4);
    CAIF_DeviceTensor scales =
        CAIF_DeviceTensor::Uninitialized({static_cast<uint32_t>(groups)}, stream, E::Float16);
    CAIF_CheckCaifq(caifq_quantize_int4_per_group(static_cast<const float *>(src_f32),
                                                  static_cast<uint8_t *>(codes.DeviceDataRaw()),
                                                  static_cast<uint16_t *>(scales.DeviceDataRaw()),
                                                  static_cast<int64_t>(elements),
                                                  static_cast<int32_t>(group_size), stream.Handle()),
                    "LoadFrozenLinear: quantize int4");
    std::vector<uint16_t> host(groups);
    scales.CopyToHostRaw(host.data());
    layer.LoadFromTensor(std::move(codes));
    layer.LoadScalesFromHost(host.data(), host.size() * sizeof(uint16_t));
    return;
  }
  CAIF_DeviceTensor converted = CAIF_DeviceTensor::Uninitialized(stored.Shape(), stream, want);
  CAIF_CheckCaifq(caifq_cast(stored.DeviceDataRaw(), code_of(stored.Dtype()), converted.DeviceDataRaw(), code_of(want),
                             static_cast<int64_t>(elements), stream.Handle()),
                  "LoadFrozenLinear: cast");
  layer.LoadFromTensor(std::move(converted));
}

// ------------------------------------------------ trainable parameters <-> file
// The trainable tensors of a layer (the LoRA factors of an adapter over a frozen base) under the names
// ParameterNames(prefix) gives them, in parameter order -- what a fine-tune checkpoint keeps beside the frozen
// base.  LoadParameters wants every name present with the parameter's dtype and element count.
inline void SaveParameters(const CAIF_DeviceLayer &layer, const std::string &prefix, const std::string &path,
                           const std::map<std::string, std::string> &metadata = {})
{
  const std::vector<std::string> names = layer.ParameterNames(prefix);
  auto &mutable_layer = const_cast<CAIF_DeviceLayer &>(layer);
  if (names.size() != mutable_layer.ParameterTensorCount())
  {
    THROW_CAIFE("SaveParameters: ParameterNames and ParameterTensorCount disagree");
  }
  std::vector<std::pair<std::string, const CAIF_DeviceTensor *>> list;
  for (size_t i = 0; i < names.size(); ++i)
  {
    list.emplace_back(names[i], &mutable_layer.ParameterTensor(i));
  }
  CAIF_SafeTensorsFormat().Save(path, list, metadata);
}

inline void LoadParameters(CAIF_DeviceLayer &layer, const std::string &prefix, const CAIF_SafeTensorsFile &file,
                           CAIF_CudaStream &stream)
{
  const std::vector<std::string> names = layer.ParameterNames(prefix);
  for (size_t i = 0; i < names.size(); ++i)
  {
    CAIF_DeviceTensor &dst = layer.ParameterTensor(i);
    CAIF_DeviceTensor src = file.Load(names[i], stream);
    if (src.Dtype() != dst.Dtype() || src.NumElements() != dst.NumElements())
    {
      THROW_CAIFE("LoadParameters: tensor '" + names[i] + "' does not match the parameter's dtype and size");
    }
    dst.CopyFromDeviceRaw(src.DeviceDataRaw(), dst.SizeBytes());
    CAIF_CheckCuda(cudaStreamSynchronize(stream.Handle()), "LoadParameters: sync");
  }
}

}   // namespace instance
