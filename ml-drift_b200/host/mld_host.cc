// Implementation of the host-side mirror (see mld_host.h).  All device work
// goes through the C ABI; this file only moves bytes and validates arguments.
#include "mld_host.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <map>

namespace mld_host {

namespace {

int DivideRoundUp(int a, int b) { return (a + b - 1) / b; }
int AlignByN(int a, int n) { return DivideRoundUp(a, n) * n; }

// IEEE binary16 <-> binary32, round to nearest even.
uint16_t FloatToHalf(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const int32_t exp = static_cast<int32_t>((x >> 23) & 0xFF) - 127 + 15;
  uint32_t man = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFF) == 0xFF) return static_cast<uint16_t>(sign | 0x7C00u | (man ? 0x200u : 0));
  if (exp >= 31) return static_cast<uint16_t>(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return static_cast<uint16_t>(sign);
    man |= 0x800000u;
    const int shift = 14 - exp;
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1))) ++q;
    return static_cast<uint16_t>(sign | q);
  }
  uint32_t q = (static_cast<uint32_t>(exp) << 10) | (man >> 13);
  const uint32_t rem = man & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (q & 1))) ++q;
  return static_cast<uint16_t>(sign | q);
}
float HalfToFloat(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while (!(man & 0x400u));
      bits = sign | (static_cast<uint32_t>(112 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

struct DeviceBuffer {
  void* ptr = nullptr;
  explicit DeviceBuffer(size_t bytes) {
    if (cudaMalloc(&ptr, bytes > 0 ? bytes : 16) != cudaSuccess) ptr = nullptr;
  }
  ~DeviceBuffer() {
    if (ptr) cudaFree(ptr);
  }
  DeviceBuffer(const DeviceBuffer&) = delete;
};

int ToAbiPrecision(CalculationsPrecision p) {
  switch (p) {
    case CalculationsPrecision::F32: return MLD_PRECISION_F32;
    case CalculationsPrecision::F16: return MLD_PRECISION_F16;
    case CalculationsPrecision::F32_F16: return MLD_PRECISION_F32F16;
  }
  return MLD_PRECISION_F32;
}

}  // namespace

Status Status::FromAbi(int abi_status, const char* where) {
  if (abi_status == MLD_OK) return OkStatus();
  std::string msg = std::string(where) + ": " + mld_status_string(abi_status) + " (" + mld_last_error() + ")";
  if (abi_status == MLD_INVALID_ARGUMENT) return Status(StatusCode::kInvalidArgument, msg);
  if (abi_status == MLD_UNIMPLEMENTED) return Status(StatusCode::kUnimplemented, msg);
  if (abi_status == MLD_NOT_FOUND) return Status(StatusCode::kNotFound, msg);
  return Status(StatusCode::kInternal, msg);
}

int SizeInBitsOf(DataType t) {
  switch (t) {
    case DataType::kFloat32:
    case DataType::kInt32: return 32;
    case DataType::kFloat16: return 16;
    case DataType::kInt8:
    case DataType::kUint8: return 8;
    case DataType::kUint4: return 4;
    default: return 0;
  }
}

DataType DeduceDataTypeFromPrecision(CalculationsPrecision p) {
  return p == CalculationsPrecision::F32 ? DataType::kFloat32 : DataType::kFloat16;
}

// ------------------------------------------------------------ TensorDescriptor
size_t TensorDescriptor::GetMemorySizeInBytes() const {
  const size_t elems = static_cast<size_t>(AlignByN(shape_.c, 4)) * shape_.b * shape_.h * shape_.w;
  return elems * SizeInBitsOf(data_type_) / 8;
}

void TensorDescriptor::UploadData(const TensorFloat32& src) {
  shape_ = src.shape;
  const int slices = DivideRoundUp(shape_.c, 4);
  const bool f16 = data_type_ == DataType::kFloat16;
  data_.assign(GetMemorySizeInBytes(), 0);
  for (int b = 0; b < shape_.b; ++b)
    for (int y = 0; y < shape_.h; ++y)
      for (int x = 0; x < shape_.w; ++x)
        for (int c = 0; c < shape_.c; ++c) {
          const float v = src.data[((static_cast<size_t>(b) * shape_.h + y) * shape_.w + x) * shape_.c + c];
          const int s = c / 4;
          // DSHWBC4 with D = 1: ((s * H + y) * W + x) * B + b) * 4 + c % 4
          const size_t idx = (((static_cast<size_t>(s) * shape_.h + y) * shape_.w + x) * shape_.b + b) * 4 + c % 4;
          (void)slices;
          if (f16)
            reinterpret_cast<uint16_t*>(data_.data())[idx] = FloatToHalf(v);
          else
            reinterpret_cast<float*>(data_.data())[idx] = v;
        }
}

void TensorDescriptor::UploadData(const Tensor<Linear, float>& src) {
  TensorFloat32 t;
  t.shape = BHWC(1, 1, 1, src.shape.v);
  t.data = src.data;
  UploadData(t);
}

void TensorDescriptor::DownloadData(TensorFloat32* dst) const {
  dst->shape = shape_;
  dst->data.assign(static_cast<size_t>(shape_.DimensionsProduct()), 0.0f);
  const bool f16 = data_type_ == DataType::kFloat16;
  for (int b = 0; b < shape_.b; ++b)
    for (int y = 0; y < shape_.h; ++y)
      for (int x = 0; x < shape_.w; ++x)
        for (int c = 0; c < shape_.c; ++c) {
          const size_t idx = (((static_cast<size_t>(c / 4) * shape_.h + y) * shape_.w + x) * shape_.b + b) * 4 + c % 4;
          const float v = f16 ? HalfToFloat(reinterpret_cast<const uint16_t*>(data_.data())[idx])
                              : reinterpret_cast<const float*>(data_.data())[idx];
          dst->data[((static_cast<size_t>(b) * shape_.h + y) * shape_.w + x) * shape_.c + c] = v;
        }
}

TensorDescriptor CreateConstantLinearTensorDescriptor(const GpuInfo&, DataType type, const Tensor<Linear, float>& src) {
  TensorDescriptor td(type, TensorStorageType::kBuffer, Layout::kLinear);
  td.SetBHWCShape(BHWC(1, 1, 1, src.shape.v));
  td.UploadData(src);
  return td;
}

TensorDescriptor ScaleOrZeroPointToTensorDesc(const GpuInfo& gpu_info, const Tensor<OHWI, float>& src,
                                              DataType dst_data_type) {
  if (src.shape.i == 1 && src.shape.h == 1) {
    Tensor<Linear, float> lin;
    lin.shape = Linear(src.shape.o);
    lin.data = src.data;
    return CreateConstantLinearTensorDescriptor(gpu_info, dst_data_type, lin);
  }
  const int O = src.shape.o, G = src.shape.i, O4 = AlignByN(O, 4);
  const bool f16 = dst_data_type == DataType::kFloat16;
  TensorDescriptor td(dst_data_type, TensorStorageType::kBuffer, Layout::kHWC);
  td.SetBHWCShape(BHWC(1, 1, DivideRoundUp(O, 4), 4 * G));  // OHIToHOIO4: HWC(1, O/4, 4*G)
  std::vector<uint8_t> out(static_cast<size_t>(G) * O4 * (f16 ? 2 : 4));
  DeviceBuffer dsrc(src.data.size() * 4), ddst(out.size());
  if (dsrc.ptr && ddst.ptr) {
    cudaMemcpy(dsrc.ptr, src.data.data(), src.data.size() * 4, cudaMemcpyHostToDevice);
    if (mld_pack_scales(static_cast<const float*>(dsrc.ptr), O, G, f16 ? 1 : 0, ddst.ptr, nullptr) == MLD_OK)
      cudaMemcpy(out.data(), ddst.ptr, out.size(), cudaMemcpyDeviceToHost);
  }
  td.UploadDataRaw(out.data(), out.size());
  return td;
}

// --------------------------------------------------------------------- packers
unsigned int GetTotalElementsCountForLayout(const WeightsDescription& desc, const OHWI& shape) {
  if (desc.layout != WeightsLayout::kOSpatialIOGroupI4O4) return static_cast<unsigned int>(-1);
  return static_cast<unsigned int>(AlignByN(shape.i, 4)) * AlignByN(shape.o, 4 * desc.GetOutputGroupSize()) * shape.h *
         shape.w;
}

TensorDescriptor GetTensorDescriptorForWeightsLayout(const Tensor<OHWI, int8_t>& weights,
                                                     const WeightsDescription& desc) {
  mld_pack_desc pd;
  std::memset(&pd, 0, sizeof pd);
  pd.o = weights.shape.o;
  pd.h = weights.shape.h;
  pd.w = weights.shape.w;
  pd.i = weights.shape.i;
  pd.bits = desc.type == DataType::kUint4 ? 4 : 8;
  pd.out_group_size = desc.GetOutputGroupSize();
  pd.source = MLD_SRC_INT8;
  pd.pad_value = pd.bits == 8 ? 128u : 8u;
  const size_t bytes = mld_packed_size_bytes(&pd);
  std::vector<uint8_t> out(bytes);
  DeviceBuffer dsrc(weights.data.size()), ddst(bytes);
  if (dsrc.ptr && ddst.ptr) {
    cudaMemcpy(dsrc.ptr, weights.data.data(), weights.data.size(), cudaMemcpyHostToDevice);
    if (mld_pack_weights(&pd, dsrc.ptr, ddst.ptr, nullptr, 0, nullptr) == MLD_OK)
      cudaMemcpy(out.data(), ddst.ptr, bytes, cudaMemcpyDeviceToHost);
  }
  TensorDescriptor td(DataType::kUint8, TensorStorageType::kBuffer, Layout::kLinear);
  td.SetBHWCShape(BHWC(1, 1, 1, static_cast<int>(bytes)));
  td.UploadDataRaw(out.data(), out.size());
  return td;
}

Status RearrangeWeightsUInt4Packed(const Tensor<OHWI, uint8_t>& weights, const WeightsDescription& desc,
                                   std::vector<uint8_t>* dst, std::vector<int32_t>* weights_sum_i,
                                   unsigned int pad_value, bool swap_dims) {
  if (desc.layout != WeightsLayout::kOSpatialIOGroupI4O4) return UnimplementedError("Unsupported layout");
  mld_pack_desc pd;
  std::memset(&pd, 0, sizeof pd);
  pd.o = weights.shape.o;
  pd.h = weights.shape.h;
  pd.w = weights.shape.w;
  pd.i = weights.shape.i;
  pd.bits = 4;
  pd.out_group_size = desc.GetOutputGroupSize();
  pd.source = MLD_SRC_UINT4_PACKED;
  pd.swap_dims = swap_dims ? 1 : 0;
  pd.pad_value = pad_value;
  const size_t bytes = mld_packed_size_bytes(&pd);
  dst->resize(bytes);
  DeviceBuffer dsrc(weights.data.size()), ddst(bytes), dsum(weights_sum_i->size() * 4);
  if (!dsrc.ptr || !ddst.ptr || !dsum.ptr) return Status(StatusCode::kInternal, "device allocation failed");
  cudaMemcpy(dsrc.ptr, weights.data.data(), weights.data.size(), cudaMemcpyHostToDevice);
  cudaMemcpy(dsum.ptr, weights_sum_i->data(), weights_sum_i->size() * 4, cudaMemcpyHostToDevice);
  const int rc = mld_pack_weights(&pd, dsrc.ptr, ddst.ptr, static_cast<int32_t*>(dsum.ptr),
                                  static_cast<int32_t>(weights_sum_i->size()), nullptr);
  if (rc != MLD_OK) return Status::FromAbi(rc, "mld_pack_weights");
  cudaMemcpy(dst->data(), ddst.ptr, bytes, cudaMemcpyDeviceToHost);
  cudaMemcpy(weights_sum_i->data(), dsum.ptr, weights_sum_i->size() * 4, cudaMemcpyDeviceToHost);
  return OkStatus();
}

Tensor<Linear, int32_t> GetWeightsAccumulatedInputChannels(const Tensor<OHWI, int8_t>& weights) {
  Tensor<Linear, int32_t> out;
  out.shape = Linear(weights.shape.o);
  out.data.assign(weights.shape.o, 0);
  DeviceBuffer dsrc(weights.data.size()), dsum(out.data.size() * 4);
  if (dsrc.ptr && dsum.ptr) {
    cudaMemcpy(dsrc.ptr, weights.data.data(), weights.data.size(), cudaMemcpyHostToDevice);
    if (mld_weights_sum_i(static_cast<const int8_t*>(dsrc.ptr), weights.shape.o,
                          weights.shape.h * weights.shape.w * weights.shape.i, static_cast<int32_t*>(dsum.ptr),
                          nullptr) == MLD_OK)
      cudaMemcpy(out.data.data(), dsum.ptr, out.data.size() * 4, cudaMemcpyDeviceToHost);
  }
  return out;
}

// -------------------------------------------------------------------- operator
WeightsDescription GetFullyConnectedInt8WeightsDesc(const GpuInfo&, const OHWI& s, bool) {
  WeightsDescription d;
  d.type = DataType::kUint8;
  d.layout = WeightsLayout::kOSpatialIOGroupI4O4;  // buffers: NVIDIA never prefers textures (fully_connected.cc:66-96)
  d.output_group_size = DivideRoundUp(s.o, 4);
  return d;
}
WeightsDescription GetFullyConnectedInt4WeightsDesc(const GpuInfo&, const OHWI& s, bool) {
  WeightsDescription d;
  d.type = DataType::kUint4;
  d.layout = WeightsLayout::kOSpatialIOGroupI4O4;
  d.output_group_size = DivideRoundUp(s.o, 4);
  return d;
}

int GetRecommendedMaxTotalSpatialSize(const GpuInfo&, CalculationsPrecision precision) {
  int base = 4;
  if (precision == CalculationsPrecision::F16) base *= 2;
  base *= 2;  // not Mali
  return base < 16 ? base : 16;
}

bool IsFullyConnectedRecommended(const GpuInfo& gpu_info, CalculationsPrecision precision, const OHWI& weights_shape,
                                 const BHWC& dst_shape) {
  int total = dst_shape.b * dst_shape.w;
  if (weights_shape.h == 1) total *= dst_shape.h;
  return total <= GetRecommendedMaxTotalSpatialSize(gpu_info, precision);
}

FullyConnected::FullyConnected(FullyConnected&& o) noexcept : GPUOperation(std::move(o)) {
  plan_ = o.plan_;
  o.plan_ = nullptr;
  has_scale_ = o.has_scale_;
  has_zp_ = o.has_zp_;
  has_bias_ = o.has_bias_;
}
FullyConnected& FullyConnected::operator=(FullyConnected&& o) noexcept {
  if (this != &o) {
    if (plan_) mld_fc_plan_destroy(plan_);
    GPUOperation::operator=(std::move(o));
    plan_ = o.plan_;
    o.plan_ = nullptr;
    has_scale_ = o.has_scale_;
    has_zp_ = o.has_zp_;
    has_bias_ = o.has_bias_;
  }
  return *this;
}
FullyConnected::~FullyConnected() {
  if (plan_) mld_fc_plan_destroy(plan_);
}

Status FullyConnected::Dispatch(const std::vector<const void*>& src, const std::vector<void*>& dst,
                                const BHWC& src_shape, void* stream) {
  size_t need = 2 + (has_scale_ ? 1 : 0) + (has_zp_ ? 1 : 0) + (has_bias_ ? 1 : 0);
  if (src.size() != need || dst.size() != 1) return InvalidArgumentError("wrong number of bound tensors");
  size_t k = 2;
  const void* scale = has_scale_ ? src[k++] : nullptr;
  const void* zp = has_zp_ ? src[k++] : nullptr;
  const void* bias = has_bias_ ? src[k++] : nullptr;
  const int tokens = src_shape.b * src_shape.h * src_shape.w;
  return Status::FromAbi(mld_fc_run(plan_, src[0], src[1], scale, zp, bias, dst[0], tokens, stream), "mld_fc_run");
}

StatusOr<FullyConnected> CreateFullyConnectedExternalWeights(const GpuInfo& gpu_info, CalculationsPrecision precision,
                                                             const TensorDescriptor& src, const TensorDescriptor& dst,
                                                             const ExternalWeights& weights,
                                                             const TensorDescriptor* bias, const BHWC* dst_shape_ptr,
                                                             int force_path) {
  const WeightsDescription& wd = weights.desc;
  if (wd.type != DataType::kUint8 && wd.type != DataType::kUint4)
    return InvalidArgumentError("Unsupported WeightsDescription type.");
  if (wd.layout != WeightsLayout::kOSpatialIOGroupI4O4)
    return InvalidArgumentError("Unsupported WeightsDescription layout: only kOSpatialIOGroupI4O4 buffers");
  if (wd.output_group_size != DivideRoundUp(weights.shape.o, 4))
    return InvalidArgumentError("Unsupported WeightsDescription output_group_size.");
  if (weights.shape.h != 1 || weights.shape.w != 1)
    return UnimplementedError("batched weights (shape.h != 1) are not part of this path");
  const DataType act = DeduceDataTypeFromPrecision(precision);
  if (src.GetDataType() != act || dst.GetDataType() != act)
    return InvalidArgumentError("src/dst tensor type does not match the calculation precision");
  mld_fc_desc d;
  std::memset(&d, 0, sizeof d);
  d.n = weights.shape.o;
  d.k = weights.shape.i;
  d.weight_bits = wd.type == DataType::kUint4 ? 4 : 8;
  if (weights.scale != nullptr) {
    // fc::IsLinearQuantized / IsBlockQuantized (fully_connected_util.cc:499-513)
    d.scale_mode = weights.scale_zp_shape.i != 1 ? MLD_SCALE_BLOCK : MLD_SCALE_PER_CHANNEL;
    d.groups = weights.scale_zp_shape.i;
  } else if (weights.scalar_scale.has_value()) {
    d.scale_mode = MLD_SCALE_SCALAR;
    d.groups = 1;
    d.scalar_scale = *weights.scalar_scale;
  } else {
    return InvalidArgumentError("quantized weights need a scale tensor or a scalar scale");
  }
  d.has_zero_point = (weights.zero_point != nullptr || weights.scalar_zero_point.has_value()) ? 1 : 0;
  if (weights.scalar_zero_point.has_value()) d.scalar_zero_point = *weights.scalar_zero_point;
  d.has_bias = bias != nullptr;
  d.precision = ToAbiPrecision(precision);
  d.src_layout = d.dst_layout = MLD_LAYOUT_SLICED;
  d.max_tokens = dst_shape_ptr ? dst_shape_ptr->b * dst_shape_ptr->h * dst_shape_ptr->w : 1;
  if (d.max_tokens < 1) d.max_tokens = 1;
  d.force_path = force_path;
  d.device = gpu_info.device;
  FullyConnected op;
  const int rc = mld_fc_plan_create(&d, &op.plan_);
  if (rc != MLD_OK) return Status::FromAbi(rc, "mld_fc_plan_create");
  op.AddSrcTensor("src_tensor");
  op.AddDstTensor("dst_tensor");
  op.AddSrcTensor("weights");  // fc::AddWeightsArguments order (fully_connected_util.cc:423-487)
  if (weights.scale != nullptr) {
    op.AddSrcTensor("weights_scale");
    op.has_scale_ = true;
  }
  if (weights.zero_point != nullptr) {
    op.AddSrcTensor("weights_zero_point");
    op.has_zp_ = true;
  }
  if (bias != nullptr) {
    op.AddSrcTensor("biases");
    op.has_bias_ = true;
  }
  const uint64_t tokens = static_cast<uint64_t>(d.max_tokens);
  op.flops_ = 2ull * tokens * d.n * d.k;  // GetConvolutionFlops (common/flops_util.cc:20-25)
  op.read_size_ = static_cast<uint64_t>(d.n) * d.k * d.weight_bits / 8;
  op.write_size_ = tokens * d.n * SizeInBitsOf(act) / 8;
  return StatusOr<FullyConnected>(std::move(op));
}

// ------------------------------------------------------------ execution harness
CudaExecutionEnvironment::CudaExecutionEnvironment() {
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) == cudaSuccess) {
    gpu_info_.device = dev;
    gpu_info_.sm_count = prop.multiProcessorCount;
    gpu_info_.name = prop.name;
  }
}

std::vector<CalculationsPrecision> CudaExecutionEnvironment::GetSupportedPrecisions() const {
  return {CalculationsPrecision::F32, CalculationsPrecision::F32_F16, CalculationsPrecision::F16};
}

Status CudaExecutionEnvironment::ExecuteGPUOperation(const std::vector<TensorDescriptor*>& src_cpu,
                                                     const std::vector<TensorDescriptor*>& dst_cpu,
                                                     std::unique_ptr<GPUOperation>&& operation) {
  std::vector<std::unique_ptr<DeviceBuffer>> bufs;
  std::vector<const void*> src;
  std::vector<void*> dst;
  for (TensorDescriptor* td : src_cpu) {
    bufs.emplace_back(new DeviceBuffer(td->GetData().size()));
    if (!bufs.back()->ptr) return Status(StatusCode::kInternal, "device allocation failed");
    cudaMemcpy(bufs.back()->ptr, td->GetData().data(), td->GetData().size(), cudaMemcpyHostToDevice);
    src.push_back(bufs.back()->ptr);
  }
  for (TensorDescriptor* td : dst_cpu) {
    bufs.emplace_back(new DeviceBuffer(td->GetMemorySizeInBytes()));
    if (!bufs.back()->ptr) return Status(StatusCode::kInternal, "device allocation failed");
    cudaMemset(bufs.back()->ptr, 0, td->GetMemorySizeInBytes());
    dst.push_back(bufs.back()->ptr);
  }
  Status s = operation->Dispatch(src, dst, src_cpu[0]->GetBHWCShape(), nullptr);
  if (!s.ok()) return s;
  if (cudaDeviceSynchronize() != cudaSuccess) return Status(StatusCode::kInternal, "kernel execution failed");
  for (size_t i = 0; i < dst_cpu.size(); ++i) {
    dst_cpu[i]->MutableData().resize(dst_cpu[i]->GetMemorySizeInBytes());
    cudaMemcpy(dst_cpu[i]->MutableData().data(), dst[i], dst_cpu[i]->GetMemorySizeInBytes(), cudaMemcpyDeviceToHost);
  }
  return OkStatus();
}

// --------------------------------------------------------------- model builder
GpuModelBuilder::TensorHandle GpuModelBuilder::AddTensor(const BHWC& shape, DataType type) {
  TensorDescriptor td(type, TensorStorageType::kBuffer, Layout::kBHWC);
  td.SetBHWCShape(shape);
  tensors_.push_back(td);
  return TensorHandle{static_cast<int>(tensors_.size()) - 1, td};
}
GpuModelBuilder::TensorHandle GpuModelBuilder::AddConstTensor(const TensorDescriptor& desc) {
  tensors_.push_back(desc);
  return TensorHandle{static_cast<int>(tensors_.size()) - 1, desc};
}

StatusOr<GpuModelBuilder::TensorHandle> GpuModelBuilder::AddFcNode(const TensorHandle& src, const Weights& weights,
                                                                   const TensorHandle* biases, const char* fc_name,
                                                                   const char* prefill_name) {
  if (!weights.scale.has_value()) return InvalidArgumentError("FullyConnectedInt*ExternalWeights requires weights.scale");
  if (weights.scale_zp_shape.i <= 0) return InvalidArgumentError("requires weights.scale_zp_shape");
  BHWC dst_shape = src.tensor_desc.GetBHWCShape();
  dst_shape.c = weights.shape.o;
  TensorHandle dst = AddTensor(dst_shape, src.tensor_desc.GetDataType());
  ExternalWeights ew;
  ew.desc = weights.desc;
  ew.shape = weights.shape;
  ew.scale_zp_shape = weights.scale_zp_shape;
  ew.scale = &tensors_[weights.scale->id];
  if (weights.zero_point) ew.zero_point = &tensors_[weights.zero_point->id];
  const TensorDescriptor* bias_desc = biases ? &biases->tensor_desc : nullptr;
  const bool decode = IsFullyConnectedRecommended(gpu_info_, precision_, weights.shape, dst_shape);
  auto op = CreateFullyConnectedExternalWeights(gpu_info_, precision_, src.tensor_desc, dst.tensor_desc, ew, bias_desc,
                                                &dst_shape, decode ? 1 : 2);
  if (!op.ok()) return op.status();
  GpuNode node;
  node.name = decode ? fc_name : prefill_name;
  node.inputs = {src.id, weights.weights.id, weights.scale->id};
  if (weights.zero_point) node.inputs.push_back(weights.zero_point->id);
  if (biases) node.inputs.push_back(biases->id);
  node.outputs = {dst.id};
  node.gpu_operation = std::make_unique<FullyConnected>(std::move(*op));
  nodes_.push_back(std::move(node));
  return dst;
}

StatusOr<GpuModelBuilder::TensorHandle> GpuModelBuilder::FullyConnectedInt4ExternalWeights(const TensorHandle& src,
                                                                                            const Weights& weights,
                                                                                            const TensorHandle* biases) {
  return AddFcNode(src, weights, biases, "fc1x1_int4_weights", "fc_prefill_int4_weights_conversion_gemm");
}
StatusOr<GpuModelBuilder::TensorHandle> GpuModelBuilder::FullyConnectedInt8ExternalWeights(const TensorHandle& src,
                                                                                            const Weights& weights,
                                                                                            const TensorHandle* biases) {
  return AddFcNode(src, weights, biases, "fc1x1_int8_weights", "fc_prefill_int8_weights_conversion_gemm");
}

Status GpuModelBuilder::Run(const std::vector<std::pair<int, const TensorDescriptor*>>& feeds,
                            const std::vector<std::pair<int, TensorDescriptor*>>& fetch) {
  std::map<int, std::unique_ptr<DeviceBuffer>> dev;
  auto ensure = [&](int id) -> void* {
    auto it = dev.find(id);
    if (it != dev.end()) return it->second->ptr;
    const TensorDescriptor& td = tensors_[id];
    const size_t bytes = td.GetData().empty() ? td.GetMemorySizeInBytes() : td.GetData().size();
    auto buf = std::make_unique<DeviceBuffer>(bytes);
    if (buf->ptr && !td.GetData().empty()) cudaMemcpy(buf->ptr, td.GetData().data(), bytes, cudaMemcpyHostToDevice);
    void* p = buf->ptr;
    dev[id] = std::move(buf);
    return p;
  };
  for (const auto& f : feeds) {
    void* p = ensure(f.first);
    if (!p) return Status(StatusCode::kInternal, "device allocation failed");
    cudaMemcpy(p, f.second->GetData().data(), f.second->GetData().size(), cudaMemcpyHostToDevice);
  }
  for (GpuNode& node : nodes_) {
    std::vector<const void*> src;
    std::vector<void*> dst;
    for (int id : node.inputs) src.push_back(ensure(id));
    for (int id : node.outputs) dst.push_back(ensure(id));
    Status s = node.gpu_operation->Dispatch(src, dst, tensors_[node.inputs[0]].GetBHWCShape(), nullptr);
    if (!s.ok()) return s;
  }
  if (cudaDeviceSynchronize() != cudaSuccess) return Status(StatusCode::kInternal, "kernel execution failed");
  for (const auto& f : fetch) {
    const TensorDescriptor& td = tensors_[f.first];
    *f.second = td;
    f.second->MutableData().resize(td.GetMemorySizeInBytes());
    cudaMemcpy(f.second->MutableData().data(), ensure(f.first), td.GetMemorySizeInBytes(), cudaMemcpyDeviceToHost);
  }
  return OkStatus();
}

// ---------------------------------------------------------------- weight files
LlmFileTensorLoader::LlmFileTensorLoader(const std::string& weights_directory, const GpuInfo& gpu_info,
                                         DataType scale_data_type)
    : gpu_info_(gpu_info), scale_type_(scale_data_type) {
  mld_loader_open(weights_directory.c_str(), &loader_);
}

LlmFileTensorLoader::~LlmFileTensorLoader() { mld_loader_close(loader_); }

std::vector<float> LlmFileTensorLoader::LoadFloat32(const std::string& name, int size) {
  std::vector<float> data(size > 0 ? size : 0);
  if (mld_loader_load_float32(loader_, name.c_str(), size, data.data()) != MLD_OK) data.clear();
  return data;
}

StatusOr<LlmFileTensorLoader::Int8Weights> LlmFileTensorLoader::LoadQuantized(const std::string& tensor_name,
                                                                               const WeightsDescription& desc,
                                                                               const OHWI& shape, bool swap_dims,
                                                                               int bits) {
  if (desc.layout != WeightsLayout::kOSpatialIOGroupI4O4) return UnimplementedError("Unsupported layout");
  if (shape.h != 1 || shape.w != 1) return UnimplementedError("spatial weights are not part of this path");
  mld_pack_desc pd;
  std::memset(&pd, 0, sizeof pd);
  pd.o = shape.o;
  pd.h = pd.w = 1;
  pd.i = shape.i;
  pd.bits = bits;
  const size_t bytes = mld_packed_size_bytes(&pd);
  DeviceBuffer packed(bytes), sums(static_cast<size_t>(shape.o) * 4);
  if (!packed.ptr || !sums.ptr) return Status(StatusCode::kInternal, "device allocation failed");
  const int rc = mld_loader_load_weights(loader_, tensor_name.c_str(), bits, shape.o, shape.i, swap_dims ? 1 : 0,
                                         packed.ptr, static_cast<int32_t*>(sums.ptr), shape.o, nullptr);
  if (rc != MLD_OK) return Status::FromAbi(rc, "mld_loader_load_weights");
  Int8Weights out;
  out.weights = TensorDescriptor(desc.type, TensorStorageType::kBuffer, Layout::kLinear);
  out.weights.SetBHWCShape(BHWC(1, 1, 1, static_cast<int>(bytes * 8 / bits)));
  out.weights.MutableData().resize(bytes);
  cudaMemcpy(out.weights.MutableData().data(), packed.ptr, bytes, cudaMemcpyDeviceToHost);
  out.weights_sum_i = TensorDescriptor(DataType::kInt32, TensorStorageType::kBuffer, Layout::kLinear);
  out.weights_sum_i.SetBHWCShape(BHWC(1, 1, 1, shape.o));
  out.weights_sum_i.MutableData().resize(static_cast<size_t>(shape.o) * 4);
  cudaMemcpy(out.weights_sum_i.MutableData().data(), sums.ptr, static_cast<size_t>(shape.o) * 4, cudaMemcpyDeviceToHost);
  return out;
}

StatusOr<LlmFileTensorLoader::Int8Weights> LlmFileTensorLoader::LoadInt8Weights(const std::string& tensor_name,
                                                                                 const WeightsDescription& desc,
                                                                                 const OHWI& shape, bool swap_dims) {
  return LoadQuantized(tensor_name, desc, shape, swap_dims, 8);
}

StatusOr<LlmFileTensorLoader::Int4Weights> LlmFileTensorLoader::LoadInt4Weights(const std::string& tensor_name,
                                                                                 const WeightsDescription& desc,
                                                                                 const OHWI& shape, bool swap_dims) {
  return LoadQuantized(tensor_name, desc, shape, swap_dims, 4);
}

int LlmFileTensorLoader::GetQuantizationIGroupSize(const std::string& weights_name, const OHWI& weights_shape) const {
  return mld_loader_group_size(loader_, weights_name.c_str(), weights_shape.o, weights_shape.i);
}

StatusOr<TensorDescriptor> LlmFileTensorLoader::LoadScale(const std::string& tensor_name, const OHWI& shape) {
  const bool f16 = scale_type_ == DataType::kFloat16;
  const int o4 = (shape.o + 3) / 4 * 4, g = shape.h * shape.w * shape.i;
  const size_t bytes = static_cast<size_t>(g) * o4 * (f16 ? 2 : 4);
  DeviceBuffer dst(bytes);
  if (!dst.ptr) return Status(StatusCode::kInternal, "device allocation failed");
  const int rc = mld_loader_load_scale(loader_, tensor_name.c_str(), shape.o, g, f16 ? 1 : 0, dst.ptr, nullptr);
  if (rc != MLD_OK) return Status::FromAbi(rc, "mld_loader_load_scale");
  TensorDescriptor td(scale_type_, TensorStorageType::kBuffer, Layout::kHWC);
  td.SetBHWCShape(BHWC(1, 1, (shape.o + 3) / 4, 4 * g));  // as ScaleOrZeroPointToTensorDesc lays it out
  td.MutableData().resize(bytes);
  cudaMemcpy(td.MutableData().data(), dst.ptr, bytes, cudaMemcpyDeviceToHost);
  return td;
}

StatusOr<TensorDescriptor> LlmFileTensorLoader::LoadZeroPoint(const std::string& zero_point_name,
                                                              const std::string& scale_name, const OHWI& shape) {
  const bool f16 = scale_type_ == DataType::kFloat16;
  const int o4 = (shape.o + 3) / 4 * 4, g = shape.h * shape.w * shape.i;
  const size_t bytes = static_cast<size_t>(g) * o4 * (f16 ? 2 : 4);
  DeviceBuffer dst(bytes);
  if (!dst.ptr) return Status(StatusCode::kInternal, "device allocation failed");
  const int rc = mld_loader_load_zero_point(loader_, zero_point_name.c_str(), scale_name.c_str(), shape.o, g, f16 ? 1 : 0,
                                            dst.ptr, nullptr);
  if (rc != MLD_OK) return Status::FromAbi(rc, "mld_loader_load_zero_point");
  TensorDescriptor td(scale_type_, TensorStorageType::kBuffer, Layout::kHWC);
  td.SetBHWCShape(BHWC(1, 1, (shape.o + 3) / 4, 4 * g));  // as ScaleOrZeroPointToTensorDesc lays it out
  td.MutableData().resize(bytes);
  cudaMemcpy(td.MutableData().data(), dst.ptr, bytes, cudaMemcpyDeviceToHost);
  return td;
}

bool LlmFileTensorLoader::HasTensor(const std::string& name) const {
  return mld_loader_has_tensor(loader_, name.c_str()) != 0;
}

int LlmFileTensorLoader::GetTensorElementSizeInBits(const std::string& tensor_name, int count) {
  return mld_loader_element_bits(loader_, tensor_name.c_str(), count);
}

}  // namespace mld_host
