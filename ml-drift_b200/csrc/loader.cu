// Reads the on-disk weight files of the LLM samples and turns them into the device tensors the
// FullyConnected operator consumes: the file-reading half runs on the host, the rearrangement into the
// kOSpatialIOGroupI4O4 layout (and the per-output weight sums) in the packing kernels of this library.
//
// File set (written by ml_drift/samples/llm/extract_weights_hf.py:355-440), all raw little-endian arrays in one
// directory, named after the checkpoint's tensor keys:
//   <key>                         float32 [..], int8 [O][I], or INT4 packed two per byte, low nibble first
//                                 (pack_int4, :232-241), [O][I / 2]
//   <key>_quantized_scale         float32 [O] or [O][I / block]; or the "group header" form: int32 group size,
//                                 then int8 / int16 values in units of 1/1024
//   <key>_quantized_zp            optional, same two forms; stored times the scale
// What each entry point does follows LlmFileTensorLoader (ml_drift/samples/llm/llm_file_tensor_loader.cc:
// LoadFloat32 :150-161, LoadInt8Weights :260-302, LoadInt4WeightsFast :351-397, GetQuantizationIGroupSize
// :399-452, LoadScale :454-467, LoadZeroPoint :469-497, HasTensor :499-509, GetTensorElementSizeInBits
// :511-522), with device pointers where the reference hands tensor descriptors to a creation callback.
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "kernels.h"

struct mld_loader {
  std::string dir;
  std::mutex mu;
  std::unordered_map<std::string, int> group_size;
  std::unordered_map<std::string, long long> file_size;
  std::unordered_map<std::string, bool> present;
};

namespace {

using mld::set_last_error_text;

// Size of a file in bytes; 0 when it cannot be opened (the reference's GetFileSize, :46-55).
long long size_of_file(const std::string& path) {
  FILE* f = std::fopen(path.c_str(), "rb");
  if (f == nullptr) return 0;
  long long n = 0;
  if (std::fseek(f, 0, SEEK_END) == 0) n = std::ftell(f);
  std::fclose(f);
  return n < 0 ? 0 : n;
}

// Reads up to `bytes` bytes from `offset`; returns how many were read, -1 when the file cannot be opened.
long long read_at(const std::string& path, long long offset, void* dst, long long bytes) {
  FILE* f = std::fopen(path.c_str(), "rb");
  if (f == nullptr) return -1;
  long long got = 0;
  if (std::fseek(f, static_cast<long>(offset), SEEK_SET) == 0)
    got = static_cast<long long>(std::fread(dst, 1, static_cast<size_t>(bytes), f));
  std::fclose(f);
  return got;
}

int not_found(const char* what, const std::string& name) {
  set_last_error_text((std::string("Failed to load ") + what + ": " + name).c_str());
  return MLD_NOT_FOUND;
}

// The scale / zero-point file as floats (LoadScaleOrZeroPoint, :128-143).  The group-header form is taken
// when the first four bytes are a plausible group size and the rest is exactly one or two bytes per value
// (IsGroupedQuantization, :104-126); anything else is read as float32.  Empty result = failure.
std::vector<float> read_scale_values(const std::string& path, long long count) {
  std::vector<float> out;
  const long long size = size_of_file(path);
  bool grouped = false;
  if (size >= 4) {
    int32_t group = 0;
    if (read_at(path, 0, &group, 4) == 4 && group > 0 && group < 65536)
      grouped = (size - 4 == count) || (size - 4 == 2 * count);
  }
  if (grouped) {
    const long long each = (size - 4) / count;
    out.resize(static_cast<size_t>(count));
    if (each == 1) {
      std::vector<int8_t> raw(static_cast<size_t>(count));
      if (read_at(path, 4, raw.data(), count) != count) return {};
      for (long long i = 0; i < count; ++i) out[i] = raw[i] / 1024.0f;
    } else {
      std::vector<int16_t> raw(static_cast<size_t>(count));
      if (read_at(path, 4, raw.data(), 2 * count) != 2 * count) return {};
      for (long long i = 0; i < count; ++i) out[i] = raw[i] / 1024.0f;
    }
    return out;
  }
  out.assign(static_cast<size_t>(count), 0.0f);
  if (read_at(path, 0, out.data(), 4 * count) < 0) return {};  // a short file leaves zeros, as an ifstream read does
  return out;
}

// [o][g] floats -> the operator's [g][o4] layout on the device (mld_pack_scales), through a staging buffer.
int upload_scale_layout(const std::vector<float>& values, int o, int g, int dst_f16, void* dst, cudaStream_t stream) {
  float* staging = nullptr;
  MLD_CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&staging), values.size() * sizeof(float)));
  cudaError_t e = cudaMemcpyAsync(staging, values.data(), values.size() * sizeof(float), cudaMemcpyHostToDevice, stream);
  int rc = MLD_OK;
  if (e != cudaSuccess) {
    mld::set_last_error("scale upload", e);
    rc = MLD_CUDA_ERROR;
  } else {
    rc = mld_pack_scales(staging, o, g, dst_f16, dst, stream);
  }
  cudaStreamSynchronize(stream);  // `values` and the staging buffer go away with this call
  cudaFree(staging);
  return rc;
}

}  // namespace

extern "C" {

int mld_loader_open(const char* weights_directory, mld_loader** out) {
  MLD_REQUIRE(weights_directory != nullptr && out != nullptr, "null argument");
  mld_loader* l = new mld_loader;
  l->dir = weights_directory;  // names are appended as they are, so the directory ends in its separator
  *out = l;
  return MLD_OK;
}

int mld_loader_close(mld_loader* loader) {
  delete loader;
  return MLD_OK;
}

int mld_loader_has_tensor(mld_loader* loader, const char* name) {
  if (loader == nullptr || name == nullptr) return 0;
  std::lock_guard<std::mutex> lock(loader->mu);
  auto it = loader->present.find(name);
  if (it != loader->present.end()) return it->second ? 1 : 0;
  FILE* f = std::fopen((loader->dir + name).c_str(), "rb");
  const bool has = f != nullptr;
  if (f != nullptr) std::fclose(f);
  loader->present[name] = has;
  return has ? 1 : 0;
}

int mld_loader_element_bits(mld_loader* loader, const char* name, int64_t count) {
  if (loader == nullptr || name == nullptr || count <= 0) return 0;
  std::lock_guard<std::mutex> lock(loader->mu);
  long long size;
  auto it = loader->file_size.find(name);
  if (it != loader->file_size.end()) {
    size = it->second;
  } else {
    size = size_of_file(loader->dir + name);
    loader->file_size[name] = size;
  }
  return static_cast<int>(size * 8 / count);
}

int mld_loader_group_size(mld_loader* loader, const char* weights_name, int32_t o, int32_t i) {
  if (loader == nullptr || weights_name == nullptr || o <= 0 || i <= 0) return i;
  std::lock_guard<std::mutex> lock(loader->mu);
  auto it = loader->group_size.find(weights_name);
  if (it != loader->group_size.end()) return it->second;
  const std::string name = weights_name;
  const std::string path = loader->dir + name.substr(0, name.rfind('.')) + ".weight_quantized_scale";
  int result = i;  // no usable scale file: one group spans all inputs
  const long long size = size_of_file(path);
  bool decided = size < 4;
  if (!decided && size % 4 == 0) {  // plain float32 values: [o][i / group]
    const long long values = size / 4;
    if (values > 0 && values % o == 0) {
      const long long per_output = values / o;
      if (i % per_output == 0) {
        result = static_cast<int>(i / per_output);
        decided = true;
      }
    }
  }
  if (!decided) {  // group header, then one or two bytes per value
    int32_t group = 0;
    if (read_at(path, 0, &group, 4) == 4 && group > 0 && group <= i && i % group == 0) {
      const long long values = static_cast<long long>(o) * (i / group);
      if (size == 4 + values || size == 4 + 2 * values) result = group;
    }
  }
  loader->group_size[name] = result;
  return result;
}

int mld_loader_load_float32(mld_loader* loader, const char* name, int64_t count, float* dst) {
  MLD_REQUIRE(loader != nullptr && name != nullptr && dst != nullptr && count >= 0, "bad argument");
  std::memset(dst, 0, static_cast<size_t>(count) * sizeof(float));
  if (read_at(loader->dir + name, 0, dst, count * 4) < 0) return not_found("tensor", name);
  return MLD_OK;
}

int mld_loader_load_weights(mld_loader* loader, const char* name, int32_t bits, int32_t o, int32_t i, int32_t swap_dims,
                            void* dst, int32_t* sum_i, int32_t sum_len, void* stream_v) {
  MLD_REQUIRE(loader != nullptr && name != nullptr && dst != nullptr, "null argument");
  MLD_REQUIRE(bits == 4 || bits == 8, "bits must be 4 or 8");
  MLD_REQUIRE(o > 0 && i > 0, "bad shape");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const long long count = static_cast<long long>(o) * i;
  if (bits == 4 && count % 2 != 0) return not_found("weights", name);  // a packed file holds whole bytes
  const long long bytes = bits == 4 ? count / 2 : count;
  std::vector<uint8_t> host(static_cast<size_t>(bytes), 0);
  if (read_at(loader->dir + name, 0, host.data(), bytes) < 0) return not_found("weights", name);
  if (bits == 8 && swap_dims) {  // the file is [i][o]
    std::vector<uint8_t> t(host.size());
    for (int oo = 0; oo < o; ++oo)
      for (int ii = 0; ii < i; ++ii) t[static_cast<size_t>(oo) * i + ii] = host[static_cast<size_t>(ii) * o + oo];
    host.swap(t);
  }
  void* staging = nullptr;
  MLD_CUDA_CHECK(cudaMalloc(&staging, host.size()));
  int rc = MLD_OK;
  const cudaError_t e = cudaMemcpyAsync(staging, host.data(), host.size(), cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) {
    mld::set_last_error("weights upload", e);
    rc = MLD_CUDA_ERROR;
  } else {
    mld_pack_desc d;
    std::memset(&d, 0, sizeof d);
    d.o = o;
    d.h = d.w = 1;
    d.i = i;
    d.bits = bits;
    d.source = bits == 4 ? MLD_SRC_UINT4_PACKED : MLD_SRC_INT8;
    d.swap_dims = bits == 4 ? swap_dims : 0;
    d.pad_value = bits == 4 ? 8u : 128u;
    rc = mld_pack_weights(&d, staging, dst, sum_i, sum_len, stream);
  }
  cudaStreamSynchronize(stream);  // the host copy and the staging buffer go away with this call
  cudaFree(staging);
  return rc;
}

int mld_loader_load_scale(mld_loader* loader, const char* name, int32_t o, int32_t g, int32_t dst_f16, void* dst,
                          void* stream) {
  MLD_REQUIRE(loader != nullptr && name != nullptr && dst != nullptr && o > 0 && g > 0, "bad argument");
  const std::vector<float> values = read_scale_values(loader->dir + name, static_cast<long long>(o) * g);
  if (values.empty()) return not_found("scale", name);
  return upload_scale_layout(values, o, g, dst_f16, dst, static_cast<cudaStream_t>(stream));
}

int mld_loader_load_zero_point(mld_loader* loader, const char* zero_point_name, const char* scale_name, int32_t o,
                               int32_t g, int32_t dst_f16, void* dst, void* stream) {
  MLD_REQUIRE(loader != nullptr && zero_point_name != nullptr && scale_name != nullptr && dst != nullptr && o > 0 && g > 0,
              "bad argument");
  const long long count = static_cast<long long>(o) * g;
  std::vector<float> zp(static_cast<size_t>(count), 0.0f);  // no file: all zero
  if (mld_loader_has_tensor(loader, zero_point_name)) {
    // the file holds zero_point * scale; the operator wants it in units of the weights
    std::vector<float> stored = read_scale_values(loader->dir + zero_point_name, count);
    const std::vector<float> scale = read_scale_values(loader->dir + scale_name, count);
    if (stored.empty() || scale.empty()) return not_found("zero point", zero_point_name);
    for (long long k = 0; k < count; ++k) zp[k] = scale[k] == 0.0f ? 0.0f : stored[k] / scale[k];
  }
  return upload_scale_layout(zp, o, g, dst_f16, dst, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
