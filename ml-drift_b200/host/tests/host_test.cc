// Tests of the host-side mirror, written the way the reference writes its kernel
// tests (ml_drift/common/kernels/tests/fully_connected_test_util.cc and
// common/task/weights_conversion_test.cc): build descriptors on the CPU, create
// the operation through the factory, run it through the execution environment,
// compare with known answers.  `--cpu` runs only the checks that need no device.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../mld_host.h"

using namespace mld_host;

static int g_failed = 0;
#define EXPECT(cond)                                                         \
  do {                                                                       \
    if (!(cond)) {                                                           \
      std::printf("  FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);        \
      ++g_failed;                                                            \
    }                                                                        \
  } while (0)
#define EXPECT_NEAR(a, b, eps) EXPECT(std::fabs((a) - (b)) <= (eps))

static const char* Name(CalculationsPrecision p) {
  return p == CalculationsPrecision::F32 ? "F32" : p == CalculationsPrecision::F16 ? "F16" : "F32_F16";
}

// ------------------------------------------------------------------- CPU only
static void TestDescriptorsAndDispatchRule() {
  GpuInfo info;
  WeightsDescription d4 = GetFullyConnectedInt4WeightsDesc(info, OHWI(533, 1, 1, 171));
  EXPECT(d4.type == DataType::kUint4 && d4.layout == WeightsLayout::kOSpatialIOGroupI4O4);
  EXPECT(d4.output_group_size == 134);
  WeightsDescription d8 = GetFullyConnectedInt8WeightsDesc(info, OHWI(2048, 1, 1, 2048));
  EXPECT(d8.type == DataType::kUint8 && d8.output_group_size == 512);
  EXPECT(GetTotalElementsCountForLayout(d4, OHWI(533, 1, 1, 171)) == 536u * 172u);
  // fully_connected.cc:981-1011 on a desktop GPU: 16 tokens at F16, 8 otherwise
  EXPECT(IsFullyConnectedRecommended(info, CalculationsPrecision::F16, OHWI(8, 1, 1, 8), BHWC(1, 1, 16, 8)));
  EXPECT(!IsFullyConnectedRecommended(info, CalculationsPrecision::F16, OHWI(8, 1, 1, 8), BHWC(1, 1, 17, 8)));
  EXPECT(IsFullyConnectedRecommended(info, CalculationsPrecision::F32_F16, OHWI(8, 1, 1, 8), BHWC(1, 2, 4, 8)));
  EXPECT(!IsFullyConnectedRecommended(info, CalculationsPrecision::F32, OHWI(8, 1, 1, 8), BHWC(3, 1, 3, 8)));
}

static void TestFactoryErrors() {
  GpuInfo info;
  TensorDescriptor f16(DataType::kFloat16, TensorStorageType::kBuffer, Layout::kHWC);
  ExternalWeights w;
  w.shape = OHWI(8, 1, 1, 8);
  w.desc = GetFullyConnectedInt4WeightsDesc(info, w.shape);
  w.scalar_scale = 0.5f;
  {
    ExternalWeights bad = w;
    bad.desc.type = DataType::kFloat32;
    auto op = CreateFullyConnectedExternalWeights(info, CalculationsPrecision::F16, f16, f16, bad, nullptr, nullptr);
    EXPECT(!op.ok() && op.status().code() == StatusCode::kInvalidArgument);
  }
  {
    ExternalWeights bad = w;
    bad.desc.output_group_size = 1;  // "Unsupported WeightsDescription output_group_size."
    auto op = CreateFullyConnectedExternalWeights(info, CalculationsPrecision::F16, f16, f16, bad, nullptr, nullptr);
    EXPECT(!op.ok() && op.status().code() == StatusCode::kInvalidArgument);
  }
  {
    ExternalWeights bad = w;
    bad.desc.layout = WeightsLayout::kUnknown;
    auto op = CreateFullyConnectedExternalWeights(info, CalculationsPrecision::F16, f16, f16, bad, nullptr, nullptr);
    EXPECT(!op.ok() && op.status().code() == StatusCode::kInvalidArgument);
  }
  {
    TensorDescriptor f32(DataType::kFloat32, TensorStorageType::kBuffer, Layout::kHWC);
    auto op = CreateFullyConnectedExternalWeights(info, CalculationsPrecision::F16, f32, f16, w, nullptr, nullptr);
    EXPECT(!op.ok());
  }
}

static void TestTensorDescriptorLayout() {
  // BUFFER storage is DSHWBC4: three tokens of six channels -> [2 slices][3 tokens][4]
  TensorFloat32 t;
  t.shape = BHWC(1, 1, 3, 6);
  for (int i = 0; i < 18; ++i) t.data.push_back(static_cast<float>(i));
  TensorDescriptor td(DataType::kFloat32, TensorStorageType::kBuffer, Layout::kHWC);
  td.UploadData(t);
  EXPECT(td.GetMemorySizeInBytes() == 2 * 3 * 4 * 4);
  const float* p = reinterpret_cast<const float*>(td.GetData().data());
  EXPECT(p[0] == 0.f && p[3] == 3.f && p[4] == 6.f && p[12] == 4.f && p[13] == 5.f && p[14] == 0.f && p[16] == 10.f);
  TensorFloat32 back;
  td.DownloadData(&back);
  EXPECT(back.data == t.data);
  TensorDescriptor th(DataType::kFloat16, TensorStorageType::kBuffer, Layout::kHWC);
  th.UploadData(t);
  EXPECT(reinterpret_cast<const uint16_t*>(th.GetData().data())[3] == 0x4200);  // 3.0 in binary16
}

// ------------------------------------------------------------------ device
static TensorDescriptor MakeSrc(DataType type, const std::vector<float>& v, int tokens = 1) {
  TensorFloat32 t;
  t.shape = BHWC(1, 1, tokens, static_cast<int>(v.size()) / tokens);
  t.data = v;
  TensorDescriptor td(type, TensorStorageType::kBuffer, Layout::kHWC);
  td.UploadData(t);
  return td;
}

static std::vector<float> RunFc(CudaExecutionEnvironment& env, CalculationsPrecision precision,
                                const Tensor<OHWI, int8_t>& wq, bool int4, const Tensor<OHWI, float>* scale,
                                const Tensor<OHWI, float>* zp, std::optional<float> scalar_scale,
                                const std::vector<float>& bias, const std::vector<float>& x, int tokens = 1) {
  const DataType type = DeduceDataTypeFromPrecision(precision);
  const GpuInfo& info = env.GetGpuInfo();
  WeightsDescription desc = int4 ? GetFullyConnectedInt4WeightsDesc(info, wq.shape) : GetFullyConnectedInt8WeightsDesc(info, wq.shape);
  TensorDescriptor weights_td = GetTensorDescriptorForWeightsLayout(wq, desc);
  TensorDescriptor scale_td, zp_td, bias_td;
  ExternalWeights ew;
  ew.desc = desc;
  ew.shape = wq.shape;
  if (scale) {
    scale_td = ScaleOrZeroPointToTensorDesc(info, *scale, type);
    ew.scale = &scale_td;
    ew.scale_zp_shape = scale->shape;
  } else {
    ew.scalar_scale = scalar_scale;
  }
  if (zp) {
    zp_td = ScaleOrZeroPointToTensorDesc(info, *zp, type);
    ew.zero_point = &zp_td;
  }
  Tensor<Linear, float> b;
  b.shape = Linear(static_cast<int>(bias.size()));
  b.data = bias;
  if (!bias.empty()) bias_td = CreateConstantLinearTensorDescriptor(info, type, b);
  TensorDescriptor src_td = MakeSrc(type, x, tokens);
  TensorDescriptor dst_td(type, TensorStorageType::kBuffer, Layout::kHWC);
  dst_td.SetBHWCShape(BHWC(1, 1, tokens, wq.shape.o));
  BHWC dst_shape = dst_td.GetBHWCShape();
  auto op = CreateFullyConnectedExternalWeights(info, precision, src_td, dst_td, ew, bias.empty() ? nullptr : &bias_td,
                                                &dst_shape);
  if (!op.ok()) {
    std::printf("  factory failed: %s\n", op.status().message().c_str());
    ++g_failed;
    return {};
  }
  std::vector<TensorDescriptor*> srcs = {&src_td, &weights_td};
  if (scale) srcs.push_back(&scale_td);
  if (zp) srcs.push_back(&zp_td);
  if (!bias.empty()) srcs.push_back(&bias_td);
  Status s = env.ExecuteGPUOperation(srcs, {&dst_td}, std::make_unique<FullyConnected>(std::move(*op)));
  if (!s.ok()) {
    std::printf("  execute failed: %s\n", s.message().c_str());
    ++g_failed;
    return {};
  }
  TensorFloat32 out;
  dst_td.DownloadData(&out);
  return out.data;
}

static void TestKnownAnswers(CudaExecutionEnvironment& env) {
  for (CalculationsPrecision p : env.GetSupportedPrecisions()) {
    const bool f32 = p == CalculationsPrecision::F32;
    std::printf(" precision %s\n", Name(p));
    {  // fully_connected_test_util.cc:49-103 -> {20.5, 15.5}
      Tensor<OHWI, int8_t> w;
      w.shape = OHWI(2, 1, 1, 4);
      w.data = {2, 4, 6, 8, 10, 12, -14, 16};
      auto y = RunFc(env, p, w, false, nullptr, nullptr, 0.5f, {0.5f, -0.5f}, {0, 1, 2, 3});
      EXPECT(y.size() == 2);
      if (y.size() == 2) {
        EXPECT_NEAR(y[0], 20.5f, f32 ? 1e-6f : 1e-3f);
        EXPECT_NEAR(y[1], 15.5f, f32 ? 1e-6f : 1e-3f);
      }
    }
    {  // :105-175 -> {91.0, 26.8}
      Tensor<OHWI, int8_t> w;
      w.shape = OHWI(2, 1, 1, 8);
      w.data = {1, 1, 1, 1, 2, 2, 2, 2, 3, 3, 3, 3, 4, 4, 4, 4};
      Tensor<OHWI, float> sc;
      sc.shape = OHWI(2, 1, 1, 2);
      sc.data = {0.5f, 2.0f, 1.0f, 0.1f};
      auto y = RunFc(env, p, w, false, &sc, nullptr, std::nullopt, {0.f, 0.f}, {0, 1, 2, 3, 4, 5, 6, 7});
      if (y.size() == 2) {
        EXPECT_NEAR(y[0], 91.0f, f32 ? 1e-5f : 0.05f);
        EXPECT_NEAR(y[1], 26.8f, f32 ? 1e-5f : 0.05f);
      }
    }
    {  // :177-249 -> {509.0, -121.4}
      Tensor<OHWI, int8_t> w;
      w.shape = OHWI(2, 1, 1, 8);
      w.data = {1, 2, 3, 4, 5, 6, 7, 8, -8, -7, -6, -5, -4, -3, -2, -1};
      Tensor<OHWI, float> sc, zp;
      sc.shape = zp.shape = OHWI(2, 1, 1, 2);
      sc.data = {0.5f, 2.0f, 1.5f, 0.1f};
      zp.data = {2, -3, 1, 4};
      auto y = RunFc(env, p, w, false, &sc, &zp, std::nullopt, {0.f, 0.f}, {1, 2, 3, 4, 5, 6, 7, 8});
      if (y.size() == 2) {
        EXPECT_NEAR(y[0], 509.0f, f32 ? 1e-4f : 0.1f);
        EXPECT_NEAR(y[1], -121.4f, f32 ? 1e-4f : 0.1f);
      }
    }
    {  // :1541-1614 -> 8.0 everywhere
      Tensor<OHWI, int8_t> w;
      w.shape = OHWI(4, 1, 1, 16);
      w.data.assign(64, 1);
      Tensor<OHWI, float> sc;
      sc.shape = OHWI(4, 1, 1, 2);
      sc.data.assign(8, 0.5f);
      auto y = RunFc(env, p, w, true, &sc, nullptr, std::nullopt, {0, 0, 0, 0}, std::vector<float>(16, 1.0f));
      for (float v : y) EXPECT_NEAR(v, 8.0f, f32 ? 1e-6f : 1e-2f);
    }
  }
}

static void TestPackers() {
  // weights_conversion_test.cc:50-91
  Tensor<OHWI, uint8_t> w;
  w.shape = OHWI(4, 1, 1, 4);
  for (uint8_t i = 0; i < 8; ++i) w.data.push_back(static_cast<uint8_t>(((2 * i + 1) << 4) | (2 * i)));
  WeightsDescription desc;
  desc.type = DataType::kUint8;
  desc.output_group_size = 1;
  desc.layout = WeightsLayout::kOSpatialIOGroupI4O4;
  std::vector<uint8_t> out;
  std::vector<int32_t> sums(4, 0);
  sums[0] = 1;  // cleared by the call (:93-135)
  Status s = RearrangeWeightsUInt4Packed(w, desc, &out, &sums, 8u, false);
  EXPECT(s.ok());
  const uint8_t nib[16] = {0, 4, 8, 12, 1, 5, 9, 13, 2, 6, 10, 14, 3, 7, 11, 15};
  EXPECT(out.size() == 8);
  for (int i = 0; i < 8 && out.size() == 8; ++i) EXPECT(out[i] == static_cast<uint8_t>((nib[2 * i] | (nib[2 * i + 1] << 4)) ^ 0x88));
  EXPECT(sums == (std::vector<int32_t>{6, 22, -26, -10}));
  // :183-219: packed-source path == int8-source path
  Tensor<OHWI, int8_t> wi8;
  wi8.shape = OHWI(4, 1, 1, 4);
  wi8.data = {-8, -7, -6, -5, -4, -3, -2, -1, 0, 1, 2, 3, 4, 5, 6, 7};
  Tensor<OHWI, uint8_t> wp;
  wp.shape = wi8.shape;
  for (int i = 0; i < 8; ++i)
    wp.data.push_back(static_cast<uint8_t>(((wi8.data[2 * i + 1] & 0xF) << 4) | (wi8.data[2 * i] & 0xF)));
  std::vector<uint8_t> out2;
  std::vector<int32_t> sums2(4, 0);
  EXPECT(RearrangeWeightsUInt4Packed(wp, desc, &out2, &sums2, 8u, false).ok());
  WeightsDescription d4 = desc;
  d4.type = DataType::kUint4;
  TensorDescriptor ref = GetTensorDescriptorForWeightsLayout(wi8, d4);
  EXPECT(ref.GetData() == out2);
  EXPECT(GetWeightsAccumulatedInputChannels(wi8).data == sums2);
  desc.layout = WeightsLayout::kUnknown;
  EXPECT(RearrangeWeightsUInt4Packed(wp, desc, &out2, &sums2, 8u, false).code() == StatusCode::kUnimplemented);
}

// decode vs prefill dispatch through the builder, checked against plain arithmetic
static void TestBuilderDispatch(CudaExecutionEnvironment& env) {
  const int K = 256, N = 64;
  Tensor<OHWI, int8_t> wq;
  wq.shape = OHWI(N, 1, 1, K);
  Tensor<OHWI, float> sc;
  sc.shape = OHWI(N, 1, 1, K / 32);
  uint32_t seed = 12345;
  auto rnd = [&]() { seed = seed * 1664525u + 1013904223u; return static_cast<float>((seed >> 8) & 0xFFFF) / 65536.0f; };
  for (int i = 0; i < N * K; ++i) wq.data.push_back(static_cast<int8_t>(static_cast<int>(rnd() * 16.0f) - 8));
  for (int i = 0; i < N * K / 32; ++i) sc.data.push_back(0.01f + 0.02f * rnd());
  for (int tokens : {1, 64}) {
    GpuModelBuilder builder(env.GetGpuInfo(), CalculationsPrecision::F32_F16);
    auto src = builder.AddTensor(BHWC(1, 1, tokens, K), DataType::kFloat16);
    GpuModelBuilder::Weights w;
    w.shape = wq.shape;
    w.desc = builder.GetFullyConnectedInt4WeightsDesc(wq.shape);
    w.scale_zp_shape = sc.shape;
    w.weights = builder.AddConstTensor(GetTensorDescriptorForWeightsLayout(wq, w.desc));
    w.scale = builder.AddConstTensor(ScaleOrZeroPointToTensorDesc(env.GetGpuInfo(), sc, DataType::kFloat16));
    auto dst = builder.FullyConnectedInt4ExternalWeights(src, w, nullptr);
    EXPECT(dst.ok());
    if (!dst.ok()) continue;
    EXPECT(builder.nodes().size() == 1);
    EXPECT(builder.nodes()[0].name == (tokens == 1 ? "fc1x1_int4_weights" : "fc_prefill_int4_weights_conversion_gemm"));
    EXPECT(builder.nodes()[0].inputs.size() == 3);  // {src, weights, scale}
    std::vector<float> x;
    for (int i = 0; i < tokens * K; ++i) x.push_back(std::round((rnd() - 0.5f) * 64.0f) / 32.0f);  // exact in fp16
    TensorDescriptor feed = MakeSrc(DataType::kFloat16, x, tokens);
    TensorDescriptor out_td;
    Status s = builder.Run({{src.id, &feed}}, {{dst->id, &out_td}});
    EXPECT(s.ok());
    if (!s.ok()) {
      std::printf("  run failed: %s\n", s.message().c_str());
      continue;
    }
    TensorFloat32 y;
    out_td.DownloadData(&y);
    double max_err = 0, max_ref = 0;
    for (int m = 0; m < tokens; ++m)
      for (int n = 0; n < N; ++n) {
        double acc = 0;
        for (int k = 0; k < K; ++k) {
          // scales are stored in fp16 by the operator
          TensorFloat32 one;
          (void)one;
          acc += static_cast<double>(x[m * K + k]) * wq.data[n * K + k] * sc.data[n * (K / 32) + k / 32];
        }
        max_err = std::fmax(max_err, std::fabs(acc - y.data[m * N + n]));
        max_ref = std::fmax(max_ref, std::fabs(acc));
      }
    std::printf(" builder tokens=%d: max err %.3g of max %.3g\n", tokens, max_err, max_ref);
    EXPECT(max_err <= 3e-3 * max_ref);  // fp16 storage of scales and outputs
  }
}

// A projection built the way the samples' Linear() builds it (samples/llm/qwen3_model_builder.cc:907-945,
// llm_weights_loader.cc:29-71): bit width from the file size, group size from the scale file, weights and
// scales from the loader, one FC node; checked against plain arithmetic on the file's own bytes.
static void TestFileLoader(CudaExecutionEnvironment& env, const std::string& dir) {
  LlmFileTensorLoader loader(dir, env.GetGpuInfo(), DataType::kFloat16);
  const std::string name = "model.layers.0.mlp.down_proj.weight", scale_name = name + "_quantized_scale";
  const OHWI shape(64, 1, 1, 160);
  EXPECT(loader.HasTensor(name) && loader.HasTensor(scale_name));
  EXPECT(!loader.HasTensor("model.layers.7.mlp.down_proj.weight"));
  EXPECT(loader.GetTensorElementSizeInBits(name, 64 * 160) == 4);
  EXPECT(loader.GetTensorElementSizeInBits("model.norm.weight", 64) == 32);
  const int group = loader.GetQuantizationIGroupSize(name, shape);
  EXPECT(group == 32);
  EXPECT(loader.LoadFloat32("model.norm.weight", 64).size() == 64);
  EXPECT(loader.LoadFloat32("missing", 4).empty());
  GpuModelBuilder builder(env.GetGpuInfo(), CalculationsPrecision::F32_F16);
  GpuModelBuilder::Weights w;
  w.shape = shape;
  w.desc = builder.GetFullyConnectedInt4WeightsDesc(shape);
  w.scale_zp_shape = OHWI(shape.o, 1, 1, shape.i / group);
  {
    auto missing = loader.LoadInt4Weights("model.layers.7.mlp.down_proj.weight", w.desc, shape, false);
    EXPECT(!missing.ok() && missing.status().code() == StatusCode::kNotFound);
    auto no_scale = loader.LoadScale("model.layers.7.mlp.down_proj.weight_quantized_scale", w.scale_zp_shape);
    EXPECT(!no_scale.ok() && no_scale.status().code() == StatusCode::kNotFound);
  }
  auto i4 = loader.LoadInt4Weights(name, w.desc, shape, false);
  auto sc = loader.LoadScale(scale_name, w.scale_zp_shape);
  EXPECT(i4.ok() && sc.ok());
  if (!i4.ok() || !sc.ok()) return;
  EXPECT(i4->weights.GetData().size() == 64u * 160u / 2u);
  EXPECT(i4->weights_sum_i.GetData().size() == 64u * 4u);
  w.weights = builder.AddConstTensor(i4->weights);
  w.scale = builder.AddConstTensor(*sc);
  auto src = builder.AddTensor(BHWC(1, 1, 1, shape.i), DataType::kFloat16);
  auto dst = builder.FullyConnectedInt4ExternalWeights(src, w, nullptr);
  EXPECT(dst.ok());
  if (!dst.ok()) return;
  std::vector<float> x;
  for (int k = 0; k < shape.i; ++k) x.push_back(static_cast<float>((k * 7) % 13 - 6) / 8.0f);  // exact in fp16
  TensorDescriptor feed = MakeSrc(DataType::kFloat16, x, 1), out_td;
  Status s = builder.Run({{src.id, &feed}}, {{dst->id, &out_td}});
  EXPECT(s.ok());
  if (!s.ok()) return;
  TensorFloat32 y;
  out_td.DownloadData(&y);
  // the file's own bytes: nibbles low first, two's complement; float32 scales [o][i / 32]
  std::vector<uint8_t> raw(64 * 160 / 2);
  std::vector<float> scales(64 * 5);
  FILE* f = std::fopen((dir + name).c_str(), "rb");
  FILE* g = std::fopen((dir + scale_name).c_str(), "rb");
  EXPECT(f != nullptr && g != nullptr);
  if (f == nullptr || g == nullptr) return;
  EXPECT(std::fread(raw.data(), 1, raw.size(), f) == raw.size());
  EXPECT(std::fread(scales.data(), 4, scales.size(), g) == scales.size());
  std::fclose(f);
  std::fclose(g);
  const int32_t* sums = reinterpret_cast<const int32_t*>(i4->weights_sum_i.GetData().data());
  double max_err = 0, max_ref = 0;
  for (int n = 0; n < shape.o; ++n) {
    double acc = 0;
    int sum = 0;
    for (int k = 0; k < shape.i; ++k) {
      const int e = n * shape.i + k;
      const int nib = (raw[e / 2] >> (4 * (e & 1))) & 15;
      const int q = ((nib + 8) & 15) - 8;
      sum += q;
      acc += static_cast<double>(x[k]) * q * scales[n * 5 + k / 32];
    }
    EXPECT(sums[n] == sum);
    max_err = std::fmax(max_err, std::fabs(acc - y.data[n]));
    max_ref = std::fmax(max_ref, std::fabs(acc));
  }
  std::printf(" loaded projection: max err %.3g of max %.3g\n", max_err, max_ref);
  EXPECT(max_err <= 3e-3 * max_ref);  // fp16 storage of scales and outputs
}

int main(int argc, char** argv) {
  const bool cpu_only = argc > 1 && std::strcmp(argv[1], "--cpu") == 0;
  std::string fixture;  // --fixture <directory of converted weight files, with its separator>
  for (int a = 1; a + 1 < argc; ++a)
    if (std::strcmp(argv[a], "--fixture") == 0) fixture = argv[a + 1];
  std::printf("[host_test] descriptors and dispatch rule\n");
  TestDescriptorsAndDispatchRule();
  std::printf("[host_test] factory errors\n");
  TestFactoryErrors();
  std::printf("[host_test] tensor descriptor layout\n");
  TestTensorDescriptorLayout();
  if (!cpu_only) {
    CudaExecutionEnvironment env;
    std::printf("[host_test] device: %s (%d SMs)\n", env.GetGpuInfo().name.c_str(), env.GetGpuInfo().sm_count);
    std::printf("[host_test] packers\n");
    TestPackers();
    std::printf("[host_test] known answers\n");
    TestKnownAnswers(env);
    std::printf("[host_test] builder dispatch\n");
    TestBuilderDispatch(env);
    if (!fixture.empty()) {
      std::printf("[host_test] file loader\n");
      TestFileLoader(env, fixture);
    }
  }
  std::printf("[host_test] %s (%d failures)\n", g_failed == 0 ? "PASSED" : "FAILED", g_failed);
  return g_failed == 0 ? 0 : 1;
}
