// Host-side C++ mirror of the ML Drift interfaces the quantized FullyConnected
// path sits behind.  Names, argument meaning and error behaviour follow the
// reference (paths relative to ml_drift/), so that code written against the
// reference's FullyConnected surface reads the same here; everything below the
// surface goes through the C ABI of include/mldfc.h.
//
//   value types           common/shape.h, common/data_type.h, common/types.h,
//                         common/precision.h, common/tensor.h
//   WeightsDescription    common/task/weights_layout.h:27-93
//   TensorDescriptor      common/task/tensor_desc.h:140-225 (BUFFER storage only)
//   ExternalWeights       common/task/gpu_operation.h:354-363
//   GPUOperation          common/task/gpu_operation.h:97-200 (surface only)
//   FullyConnected & co.  common/kernels/fully_connected.h:39-161
//   packers               common/task/weights_conversion.h:35-112
//   GpuModelBuilder       common/gpu_model_builder.h:189-210 (FC entry points)
//   execution harness     common/task/testing_util.h:48-143
//   LlmFileTensorLoader   samples/llm/llm_file_tensor_loader.h:34-84
#pragma once

#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <utility>
#include <vector>

#include "mldfc.h"

namespace mld_host {

// ------------------------------------------------------------------ status
// Stand-in for absl::Status / absl::StatusOr (abseil is not a dependency here).
enum class StatusCode { kOk = 0, kInvalidArgument = 3, kNotFound = 5, kUnimplemented = 12, kInternal = 13 };
class Status {
 public:
  Status() = default;
  Status(StatusCode c, std::string m) : code_(c), message_(std::move(m)) {}
  bool ok() const { return code_ == StatusCode::kOk; }
  StatusCode code() const { return code_; }
  const std::string& message() const { return message_; }
  static Status FromAbi(int abi_status, const char* where);

 private:
  StatusCode code_ = StatusCode::kOk;
  std::string message_;
};
inline Status OkStatus() { return Status(); }
inline Status InvalidArgumentError(std::string m) { return Status(StatusCode::kInvalidArgument, std::move(m)); }
inline Status UnimplementedError(std::string m) { return Status(StatusCode::kUnimplemented, std::move(m)); }
inline Status NotFoundError(std::string m) { return Status(StatusCode::kNotFound, std::move(m)); }

template <typename T>
class StatusOr {
 public:
  StatusOr(Status s) : status_(std::move(s)) {}  // NOLINT
  StatusOr(T v) : value_(std::move(v)) {}        // NOLINT
  bool ok() const { return status_.ok(); }
  const Status& status() const { return status_; }
  T& operator*() { return *value_; }
  T* operator->() { return &*value_; }

 private:
  Status status_;
  std::optional<T> value_;
};

// -------------------------------------------------------------- value types
struct OHWI {
  int o = 0, h = 0, w = 0, i = 0;
  OHWI() = default;
  OHWI(int o_, int h_, int w_, int i_) : o(o_), h(h_), w(w_), i(i_) {}
  int64_t DimensionsProduct() const { return int64_t(o) * h * w * i; }
  int64_t LinearIndex(int oo, int hh, int ww, int ii) const { return ((int64_t(oo) * h + hh) * w + ww) * i + ii; }
};
struct BHWC {
  int b = 0, h = 0, w = 0, c = 0;
  BHWC() = default;
  BHWC(int b_, int h_, int w_, int c_) : b(b_), h(h_), w(w_), c(c_) {}
  int64_t DimensionsProduct() const { return int64_t(b) * h * w * c; }
};
struct Linear {
  int v = 0;
  Linear() = default;
  explicit Linear(int v_) : v(v_) {}
  int64_t DimensionsProduct() const { return v; }
};

enum class DataType { kUnknown, kFloat16, kFloat32, kInt8, kUint8, kUint4, kInt32 };
int SizeInBitsOf(DataType t);
enum class CalculationsPrecision { F32, F32_F16, F16 };  // common/precision.h:25-36
DataType DeduceDataTypeFromPrecision(CalculationsPrecision p);

template <typename ShapeT, typename ElemT>
struct Tensor {
  ShapeT shape;
  std::vector<ElemT> data;
  const ElemT* Data() const { return data.data(); }
};
using TensorFloat32 = Tensor<BHWC, float>;

// Identifies the one device this library targets (the reference's GpuInfo has
// ~200 vendor predicates; none of them select anything here).
struct GpuInfo {
  int device = 0;
  int sm_count = 0;
  std::string name;
  bool IsApiCuda() const { return true; }
};

// -------------------------------------------------------- weights description
enum class WeightsLayout { kUnknown, kOSpatialIOGroupI4O4 };
struct WeightsDescription {
  DataType type = DataType::kUnknown;
  WeightsLayout layout = WeightsLayout::kUnknown;
  int output_group_size = 0;
  int GetOutputGroupSize() const { return output_group_size; }
  bool IsLinearLayout() const { return layout == WeightsLayout::kOSpatialIOGroupI4O4; }
  bool IsI4O4() const { return layout == WeightsLayout::kOSpatialIOGroupI4O4; }
};

// ----------------------------------------------------------- tensor descriptor
enum class TensorStorageType { kUnknown, kBuffer };
enum class Layout { kUnknown, kLinear, kHWC, kBHWC };

// Host-side container of one tensor in device layout (BUFFER storage:
// [ceil(C/4)][B*H*W][4] for spatial tensors, padded vectors for linear ones).
class TensorDescriptor {
 public:
  TensorDescriptor() = default;
  TensorDescriptor(DataType t, TensorStorageType s, Layout l) : data_type_(t), storage_(s), layout_(l) {}
  DataType GetDataType() const { return data_type_; }
  TensorStorageType GetStorageType() const { return storage_; }
  Layout GetLayout() const { return layout_; }
  void SetBHWCShape(const BHWC& s) { shape_ = s; }
  BHWC GetBHWCShape() const { return shape_; }
  size_t GetMemorySizeInBytes() const;
  // logical floats <-> device layout (f32 -> f16 round-to-nearest-even when the descriptor is fp16)
  void UploadData(const TensorFloat32& src);
  void UploadData(const Tensor<Linear, float>& src);
  void DownloadData(TensorFloat32* dst) const;
  void UploadDataRaw(const uint8_t* bytes, size_t n) { data_.assign(bytes, bytes + n); }
  const std::vector<uint8_t>& GetData() const { return data_; }
  std::vector<uint8_t>& MutableData() { return data_; }

 private:
  DataType data_type_ = DataType::kUnknown;
  TensorStorageType storage_ = TensorStorageType::kUnknown;
  Layout layout_ = Layout::kUnknown;
  BHWC shape_;
  std::vector<uint8_t> data_;
};

TensorDescriptor CreateConstantLinearTensorDescriptor(const GpuInfo&, DataType, const Tensor<Linear, float>& src);
// common/task/tensor_desc.cc:2245-2257; runs mld_pack_scales on the device.
TensorDescriptor ScaleOrZeroPointToTensorDesc(const GpuInfo&, const Tensor<OHWI, float>& src, DataType dst_data_type);

// ------------------------------------------------------------------- packers
unsigned int GetTotalElementsCountForLayout(const WeightsDescription&, const OHWI& shape);
// GetTensorDescriptorForWeightsLayout(int8) (weights_conversion.cc:1672-1713): CUDA packing kernel.
TensorDescriptor GetTensorDescriptorForWeightsLayout(const Tensor<OHWI, int8_t>& weights, const WeightsDescription&);
// RearrangeWeightsUInt4Packed (weights_conversion.cc:1604-1620).  dst / weights_sum_i are host spans.
Status RearrangeWeightsUInt4Packed(const Tensor<OHWI, uint8_t>& weights, const WeightsDescription& dst_weight_desc,
                                   std::vector<uint8_t>* dst, std::vector<int32_t>* weights_sum_i,
                                   unsigned int pad_value, bool swap_dims);
Tensor<Linear, int32_t> GetWeightsAccumulatedInputChannels(const Tensor<OHWI, int8_t>& weights);

// ------------------------------------------------------------------ operator
struct ExternalWeights {
  WeightsDescription desc;
  OHWI shape;
  OHWI scale_zp_shape = OHWI(1, 1, 1, 1);
  const TensorDescriptor* scale = nullptr;
  const TensorDescriptor* zero_point = nullptr;
  std::optional<float> scalar_scale;
  std::optional<float> scalar_zero_point;
};

class GPUOperation {
 public:
  virtual ~GPUOperation() = default;
  GPUOperation() = default;
  GPUOperation(GPUOperation&&) = default;
  GPUOperation& operator=(GPUOperation&&) = default;
  GPUOperation(const GPUOperation&) = delete;
  // Tensors are referenced by name and positional order, as in the reference.
  const std::vector<std::string>& GetSrcTensorsNames() const { return src_names_; }
  const std::vector<std::string>& GetDstTensorsNames() const { return dst_names_; }
  // Enqueues the operation; src/dst are device pointers in src/dst name order.
  virtual Status Dispatch(const std::vector<const void*>& src, const std::vector<void*>& dst, const BHWC& src_shape,
                          void* stream) = 0;
  uint64_t flops_ = 0, read_size_ = 0, write_size_ = 0;

 protected:
  void AddSrcTensor(const std::string& name) { src_names_.push_back(name); }
  void AddDstTensor(const std::string& name) { dst_names_.push_back(name); }

 private:
  std::vector<std::string> src_names_, dst_names_;
};

WeightsDescription GetFullyConnectedInt8WeightsDesc(const GpuInfo&, const OHWI& weights_shape,
                                                    bool prefer_textures = false);
WeightsDescription GetFullyConnectedInt4WeightsDesc(const GpuInfo&, const OHWI& weights_shape,
                                                    bool prefer_textures = false);
int GetRecommendedMaxTotalSpatialSize(const GpuInfo&, CalculationsPrecision);
bool IsFullyConnectedRecommended(const GpuInfo&, CalculationsPrecision, const OHWI& weights_shape,
                                 const BHWC& dst_shape);

class FullyConnected : public GPUOperation {
 public:
  FullyConnected() = default;
  FullyConnected(FullyConnected&&) noexcept;
  FullyConnected& operator=(FullyConnected&&) noexcept;
  ~FullyConnected() override;
  Status Dispatch(const std::vector<const void*>& src, const std::vector<void*>& dst, const BHWC& src_shape,
                  void* stream) override;
  bool has_scale_tensor() const { return has_scale_; }
  bool has_zero_point_tensor() const { return has_zp_; }
  bool has_bias() const { return has_bias_; }

 private:
  friend StatusOr<FullyConnected> CreateFullyConnectedExternalWeights(const GpuInfo&, CalculationsPrecision,
                                                                      const TensorDescriptor&, const TensorDescriptor&,
                                                                      const ExternalWeights&, const TensorDescriptor*,
                                                                      const BHWC*, int);
  mld_fc_plan* plan_ = nullptr;
  bool has_scale_ = false, has_zp_ = false, has_bias_ = false;
};

// common/kernels/fully_connected.h:155-161.  dst_shape_ptr bounds the token
// count the operator will see (B*H*W); force_path: 0 = the reference's rule.
StatusOr<FullyConnected> CreateFullyConnectedExternalWeights(const GpuInfo& gpu_info, CalculationsPrecision precision,
                                                             const TensorDescriptor& src, const TensorDescriptor& dst,
                                                             const ExternalWeights& weights,
                                                             const TensorDescriptor* bias, const BHWC* dst_shape_ptr,
                                                             int force_path = 0);

// ---------------------------------------------------------- execution harness
// Shape of TestExecutionEnvironment (common/task/testing_util.h:48-143) and of
// its OpenCL implementation (cl/testing/cl_test.cc:63-91): create device tensors
// from CPU descriptors, bind, dispatch, wait, download.
class CudaExecutionEnvironment {
 public:
  CudaExecutionEnvironment();
  const GpuInfo& GetGpuInfo() const { return gpu_info_; }
  std::vector<CalculationsPrecision> GetSupportedPrecisions() const;
  std::vector<TensorStorageType> GetSupportedStorages() const { return {TensorStorageType::kBuffer}; }
  Status ExecuteGPUOperation(const std::vector<TensorDescriptor*>& src_cpu, const std::vector<TensorDescriptor*>& dst_cpu,
                             std::unique_ptr<GPUOperation>&& operation);

 private:
  GpuInfo gpu_info_;
};

// ------------------------------------------------------------- model builder
// The FullyConnected entry points of GpuModelBuilder
// (common/gpu_model_builder.cc:1548-1725) and the node container of
// common/gpu_model.h:38-60.
struct GpuNode {
  std::unique_ptr<GPUOperation> gpu_operation;
  std::vector<int> inputs, outputs;
  std::string name;
};

class GpuModelBuilder {
 public:
  struct TensorHandle {
    int id = -1;
    TensorDescriptor tensor_desc;
  };
  struct Weights {  // common/gpu_model_builder.h:66-75
    WeightsDescription desc;
    OHWI shape;
    OHWI scale_zp_shape = OHWI(1, 1, 1, 1);
    TensorHandle weights;
    std::optional<TensorHandle> scale, zero_point, sum_i;
  };
  GpuModelBuilder(const GpuInfo& gpu_info, CalculationsPrecision precision) : gpu_info_(gpu_info), precision_(precision) {}
  TensorHandle AddTensor(const BHWC& shape, DataType type);
  TensorHandle AddConstTensor(const TensorDescriptor& desc);
  WeightsDescription GetFullyConnectedInt4WeightsDesc(const OHWI& s) { return mld_host::GetFullyConnectedInt4WeightsDesc(gpu_info_, s); }
  WeightsDescription GetFullyConnectedInt8WeightsDesc(const OHWI& s) { return mld_host::GetFullyConnectedInt8WeightsDesc(gpu_info_, s); }
  // Append one FC node with inputs {src, weights, scale, [zp], [bias]} (decode
  // kernel when IsFullyConnectedRecommended, otherwise the prefill GEMM).
  StatusOr<TensorHandle> FullyConnectedInt4ExternalWeights(const TensorHandle& src, const Weights& weights,
                                                           const TensorHandle* biases);
  StatusOr<TensorHandle> FullyConnectedInt8ExternalWeights(const TensorHandle& src, const Weights& weights,
                                                           const TensorHandle* biases);
  const std::vector<GpuNode>& nodes() const { return nodes_; }
  std::vector<GpuNode>& mutable_nodes() { return nodes_; }
  const std::vector<TensorDescriptor>& tensors() const { return tensors_; }
  // Runs the nodes in order on the device: uploads `feeds` (tensor id -> descriptor with data),
  // dispatches every node, downloads `fetch` ids.
  Status Run(const std::vector<std::pair<int, const TensorDescriptor*>>& feeds,
             const std::vector<std::pair<int, TensorDescriptor*>>& fetch);

 private:
  StatusOr<TensorHandle> AddFcNode(const TensorHandle& src, const Weights& weights, const TensorHandle* biases,
                                   const char* fc_name, const char* prefill_name);
  GpuInfo gpu_info_;
  CalculationsPrecision precision_;
  std::vector<TensorDescriptor> tensors_;
  std::vector<GpuNode> nodes_;
};

// ------------------------------------------------------------- weight files
// LlmFileTensorLoader (samples/llm/llm_file_tensor_loader.h:34-84) over mld_loader_*: reads the converter's
// files and returns tensors in device layout.  Where the reference hands each descriptor to the tensor-creation
// callback of its model builder, this returns the descriptor (GpuModelBuilder::AddConstTensor takes it).
class LlmFileTensorLoader {
 public:
  struct Int8Weights {  // samples/llm/llm_tensor_loader.h: weights + weights_sum_i
    TensorDescriptor weights;
    TensorDescriptor weights_sum_i;
  };
  using Int4Weights = Int8Weights;
  // scale_data_type: the type scales and zero points are stored in (the builder's activation type)
  LlmFileTensorLoader(const std::string& weights_directory, const GpuInfo& gpu_info, DataType scale_data_type);
  ~LlmFileTensorLoader();
  LlmFileTensorLoader(const LlmFileTensorLoader&) = delete;
  LlmFileTensorLoader& operator=(const LlmFileTensorLoader&) = delete;

  std::vector<float> LoadFloat32(const std::string& name, int size);  // empty when the file is missing
  StatusOr<Int8Weights> LoadInt8Weights(const std::string& tensor_name, const WeightsDescription& weights_desc,
                                        const OHWI& shape, bool swap_dims);
  StatusOr<Int4Weights> LoadInt4Weights(const std::string& tensor_name, const WeightsDescription& weights_desc,
                                        const OHWI& shape, bool swap_dims);
  int GetQuantizationIGroupSize(const std::string& weights_name, const OHWI& weights_shape) const;
  StatusOr<TensorDescriptor> LoadScale(const std::string& tensor_name, const OHWI& shape);
  StatusOr<TensorDescriptor> LoadZeroPoint(const std::string& zero_point_name, const std::string& scale_name,
                                           const OHWI& shape);
  bool HasTensor(const std::string& name) const;
  int GetTensorElementSizeInBits(const std::string& tensor_name, int count);

 private:
  StatusOr<Int8Weights> LoadQuantized(const std::string& tensor_name, const WeightsDescription& weights_desc,
                                      const OHWI& shape, bool swap_dims, int bits);
  mld_loader* loader_ = nullptr;
  GpuInfo gpu_info_;
  DataType scale_type_;
};

}  // namespace mld_host
