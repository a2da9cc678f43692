// GPU exercise of the C++ drop-in API, written after the reference's own GPU
// tests (same inputs, tolerances and checks), with cuda_bf16.h standing in for
// the CUTLASS host BF16 type:
//   grouped  baselines/cutlass/test_correctness.cu:60-157   tokens {7,0,13,31}, N=K=32
//   dense    tests/test_sm100_dense_correctness.cu:55-129   128 x 128 x 64
//   pair     tests/test_sm100_2sm_correctness.cu:55-128     256 x 128 x 64
//   direct   tests/test_direct_cute_correctness.cu:55-126   128 x 256 x 64, FP32 out
//   probe    tests/test_scheduler_probe.cu:100-128          37 tiles, 8 CTAs
// plus one case of the FP8 E4M3 plan, which the reference does not have.
// Prints "SKIP" and exits 0 on a device that is not compute capability 10.0.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <numeric>
#include <stdexcept>
#include <string>
#include <vector>

#include "blackwell_moe/kernels/direct_cute_gemm.cuh"
#include "blackwell_moe/kernels/grouped_gemm.cuh"
#include "blackwell_moe/kernels/sm100_2sm_gemm.cuh"
#include "blackwell_moe/kernels/sm100_dense_gemm.cuh"
#include "blackwell_moe/scheduler/scheduler_probe.cuh"

using namespace blackwell_moe;

namespace {

void require(bool ok, const std::string& what) {
  if (!ok) throw std::runtime_error(what);
}
void cuda_ok(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <class T>
struct Dev {
  T* p = nullptr;
  explicit Dev(size_t n) { cuda_ok(cudaMalloc(reinterpret_cast<void**>(&p), n * sizeof(T)), "cudaMalloc"); }
  ~Dev() { cudaFree(p); }
  void upload(const std::vector<T>& h) {
    cuda_ok(cudaMemcpy(p, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice), "H2D");
  }
  std::vector<T> download(size_t n) const {
    std::vector<T> h(n);
    cuda_ok(cudaMemcpy(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost), "D2H");
    return h;
  }
};

std::vector<__nv_bfloat16> fill(size_t n, int mul, int add, int mod, int off, float div) {
  std::vector<__nv_bfloat16> v(n);
  for (size_t i = 0; i < n; ++i) {
    const int x = static_cast<int>((i * mul + add) % mod) - off;
    v[i] = __float2bfloat16(static_cast<float>(x) / div);
  }
  return v;
}

float ref_dot(const std::vector<__nv_bfloat16>& a, const std::vector<__nv_bfloat16>& b,
              uint32_t row, uint32_t col, uint32_t k) {
  float acc = 0.0f;
  for (uint32_t i = 0; i < k; ++i) {
    acc += __bfloat162float(a[static_cast<size_t>(row) * k + i]) *
           __bfloat162float(b[static_cast<size_t>(col) * k + i]);
  }
  return acc;
}

void grouped_kat() {
  const std::vector<uint32_t> tokens{7, 0, 13, 31};
  const uint32_t n = 32, k = 32;
  std::vector<std::vector<__nv_bfloat16>> ha(4), hb(4);
  std::vector<Dev<__nv_bfloat16>*> da(4, nullptr), db(4, nullptr), dd(4, nullptr);
  std::vector<const void*> pa(4, nullptr), pb(4, nullptr);
  std::vector<void*> pd(4, nullptr);
  for (uint32_t e = 0; e < 4; ++e) {
    if (tokens[e] == 0) continue;
    ha[e] = fill(static_cast<size_t>(tokens[e]) * k, 1, 3 * e, 11, 5, 8.0f);
    hb[e] = fill(static_cast<size_t>(n) * k, 3, e, 13, 6, 8.0f);
    da[e] = new Dev<__nv_bfloat16>(ha[e].size());
    db[e] = new Dev<__nv_bfloat16>(hb[e].size());
    dd[e] = new Dev<__nv_bfloat16>(static_cast<size_t>(tokens[e]) * n);
    da[e]->upload(ha[e]);
    db[e]->upload(hb[e]);
    cuda_ok(cudaMemset(dd[e]->p, 0, static_cast<size_t>(tokens[e]) * n * 2), "memset");
    pa[e] = da[e]->p; pb[e] = db[e]->p; pd[e] = dd[e]->p;
  }
  GroupedGemmArguments args;
  args.a = pa.data(); args.b = pb.data(); args.d = pd.data();
  args.tokens_per_expert = tokens.data();
  args.experts = 4; args.n = n; args.k = k;
  for (SchedulerKind policy : {SchedulerKind::kExpertOrder, SchedulerKind::kStaticPersistent,
                               SchedulerKind::kDynamicQueue, SchedulerKind::kCompacted,
                               SchedulerKind::kAuto, SchedulerKind::kClc}) {
    args.scheduler = policy;
    Bf16GroupedGemmPlan plan;
    KernelStatus st = plan.initialize(args);
    require(st == KernelStatus::kSuccess, kernel_status_string(st));
    require(plan.stats().active_experts == 3, "inactive expert filtering is incorrect");
    st = plan.run();
    require(st == KernelStatus::kSuccess, kernel_status_string(st));
    require(plan.poll() == KernelStatus::kSuccess, "device status");
    for (uint32_t e = 0; e < 4; ++e) {
      if (tokens[e] == 0) continue;
      const auto out = dd[e]->download(static_cast<size_t>(tokens[e]) * n);
      for (uint32_t r = 0; r < tokens[e]; ++r) {
        for (uint32_t c = 0; c < n; ++c) {
          const float ref = ref_dot(ha[e], hb[e], r, c, k);
          const float got = __bfloat162float(out[r * n + c]);
          require(std::fabs(got - ref) <= 0.08f + 0.02f * std::fabs(ref),
                  "grouped GEMM result exceeds tolerance (" + to_string(policy) + ")");
        }
      }
    }
  }
  // argument contract of the reference plan
  GroupedGemmArguments bad = args;
  bad.n = 30;
  Bf16GroupedGemmPlan plan;
  require(plan.initialize(bad) == KernelStatus::kInvalidArgument, "n % 8 must be rejected");
  bad = args; bad.data_type = DataType::kFp8E4M3;
  require(plan.initialize(bad) == KernelStatus::kUnsupportedDataType, "FP8 must be rejected");
  require(plan.run() == KernelStatus::kInvalidArgument, "run() after failed initialize()");
  require(launch_grouped_gemm_baseline(args) == KernelStatus::kSuccess, "one-shot launch");
  for (uint32_t e = 0; e < 4; ++e) { delete da[e]; delete db[e]; delete dd[e]; }
}

// FP8 E4M3 plan (an extension: the reference only declares the type). Operands are
// multiples of 1/8 of magnitude <= 5/8, which E4M3 holds exactly; every product is a
// multiple of 1/64 and the sums of k = 160 of them are exact in FP32, so the expected
// output is the exact sum rounded once to BF16 and the comparison is bitwise.
void fp8_kat() {
  const std::vector<uint32_t> tokens{7, 0, 13, 131};
  const uint32_t n = 40, k = 160;
  auto fill8 = [](size_t count, int mul, int add, int mod, int off) {
    std::vector<__nv_fp8_e4m3> v(count);
    for (size_t i = 0; i < count; ++i) {
      v[i] = __nv_fp8_e4m3(static_cast<float>(static_cast<int>((i * mul + add) % mod) - off) / 8.0f);
    }
    return v;
  };
  std::vector<std::vector<__nv_fp8_e4m3>> ha(4), hb(4);
  std::vector<Dev<__nv_fp8_e4m3>*> da(4, nullptr), db(4, nullptr);
  std::vector<Dev<__nv_bfloat16>*> dd(4, nullptr);
  std::vector<const void*> pa(4, nullptr), pb(4, nullptr);
  std::vector<void*> pd(4, nullptr);
  for (uint32_t e = 0; e < 4; ++e) {
    if (tokens[e] == 0) continue;
    ha[e] = fill8(static_cast<size_t>(tokens[e]) * k, 1, 3 * e, 11, 5);
    hb[e] = fill8(static_cast<size_t>(n) * k, 3, e, 9, 4);
    da[e] = new Dev<__nv_fp8_e4m3>(ha[e].size());
    db[e] = new Dev<__nv_fp8_e4m3>(hb[e].size());
    dd[e] = new Dev<__nv_bfloat16>(static_cast<size_t>(tokens[e]) * n);
    da[e]->upload(ha[e]);
    db[e]->upload(hb[e]);
    pa[e] = da[e]->p; pb[e] = db[e]->p; pd[e] = dd[e]->p;
  }
  GroupedGemmArguments args;
  args.a = pa.data(); args.b = pb.data(); args.d = pd.data();
  args.tokens_per_expert = tokens.data();
  args.experts = 4; args.n = n; args.k = k;
  args.data_type = DataType::kFp8E4M3;
  for (SchedulerKind policy : {SchedulerKind::kExpertOrder, SchedulerKind::kDynamicQueue,
                               SchedulerKind::kClc}) {
    for (uint32_t group : {1u, 2u}) {
      args.scheduler = policy;
      args.cta_group = group;
      for (uint32_t e = 0; e < 4; ++e) {
        if (tokens[e] != 0) {
          cuda_ok(cudaMemset(dd[e]->p, 0xff, static_cast<size_t>(tokens[e]) * n * 2), "memset");
        }
      }
      Fp8E4m3GroupedGemmPlan plan;
      KernelStatus st = plan.initialize(args);
      require(st == KernelStatus::kSuccess, std::string("FP8: ") + kernel_status_string(st));
      require(plan.run() == KernelStatus::kSuccess, "FP8 run");
      require(plan.poll() == KernelStatus::kSuccess, "FP8 device status");
      for (uint32_t e = 0; e < 4; ++e) {
        if (tokens[e] == 0) continue;
        const auto out = dd[e]->download(static_cast<size_t>(tokens[e]) * n);
        for (uint32_t r = 0; r < tokens[e]; ++r) {
          for (uint32_t c = 0; c < n; ++c) {
            float acc = 0.0f;
            for (uint32_t i = 0; i < k; ++i) {
              acc += static_cast<float>(ha[e][static_cast<size_t>(r) * k + i]) *
                     static_cast<float>(hb[e][static_cast<size_t>(c) * k + i]);
            }
            const __nv_bfloat16 want = __float2bfloat16(acc);
            const __nv_bfloat16 got = out[r * n + c];
            require(__bfloat162float(got) == __bfloat162float(want),
                    "FP8 grouped GEMM differs from the exact result");
          }
        }
      }
    }
  }
  Fp8E4m3GroupedGemmPlan plan;
  GroupedGemmArguments bad = args;
  bad.data_type = DataType::kBf16;
  require(plan.initialize(bad) == KernelStatus::kUnsupportedDataType, "FP8 plan takes FP8 only");
  bad = args; bad.k = 40;
  require(plan.initialize(bad) == KernelStatus::kInvalidArgument, "k % 16 must be rejected");
  for (uint32_t e = 0; e < 4; ++e) { delete da[e]; delete db[e]; delete dd[e]; }
}

template <class Plan>
void dense_kat(uint32_t m, uint32_t n, uint32_t k, int a_mod, int a_off, int b_mul, int b_mod,
               int b_off, const char* what) {
  const auto ha = fill(static_cast<size_t>(m) * k, 1, 0, a_mod, a_off, 16.0f);
  const auto hb = fill(static_cast<size_t>(n) * k, b_mul, 0, b_mod, b_off, 16.0f);
  Dev<__nv_bfloat16> a(ha.size()), b(hb.size()), d(static_cast<size_t>(m) * n);
  a.upload(ha); b.upload(hb);
  cuda_ok(cudaMemset(d.p, 0, static_cast<size_t>(m) * n * 2), "memset");
  Sm100DenseGemmArguments args;
  args.a = a.p; args.b = b.p; args.d = d.p; args.m = m; args.n = n; args.k = k;
  Plan plan;
  KernelStatus st = plan.initialize(args);
  require(st == KernelStatus::kSuccess, std::string(what) + ": " + kernel_status_string(st));
  require(plan.stats().persistent_ctas > 0 && plan.stats().sm_count > 0, "plan stats");
  st = plan.run();
  require(st == KernelStatus::kSuccess, kernel_status_string(st));
  cuda_ok(cudaDeviceSynchronize(), what);
  const auto out = d.download(static_cast<size_t>(m) * n);
  for (uint32_t r = 0; r < m; ++r) {
    for (uint32_t c = 0; c < n; ++c) {
      const float ref = ref_dot(ha, hb, r, c, k);
      const float got = __bfloat162float(out[static_cast<size_t>(r) * n + c]);
      require(std::fabs(got - ref) <= 0.04f + 0.02f * std::fabs(ref),
              std::string(what) + " exceeds tolerance");
    }
  }
  Sm100DenseGemmArguments bad = args;
  bad.k = 60;
  require(plan.initialize(bad) == KernelStatus::kInvalidArgument, "k % 8 must be rejected");
}

void direct_kat() {
  const uint32_t m = 128, n = 256, k = 64;
  const auto ha = fill(static_cast<size_t>(m) * k, 1, 0, 9, 4, 16.0f);
  const auto hb = fill(static_cast<size_t>(n) * k, 3, 0, 11, 5, 16.0f);
  Dev<__nv_bfloat16> a(ha.size()), b(hb.size());
  Dev<float> d(static_cast<size_t>(m) * n);
  a.upload(ha); b.upload(hb);
  cuda_ok(cudaMemset(d.p, 0, static_cast<size_t>(m) * n * 4), "memset");
  DirectCuteGemmArguments args;
  args.a = a.p; args.b = b.p; args.d = d.p; args.m = m; args.n = n; args.k = k;
  DirectCuteGemmStats stats;
  const KernelStatus st = launch_direct_cute_gemm(args, &stats);
  require(st == KernelStatus::kSuccess, std::string("direct: ") + kernel_status_string(st));
  require(stats.grid_m == 1 && stats.grid_n == 1 && stats.dynamic_smem_bytes > 0, "direct stats");
  cuda_ok(cudaDeviceSynchronize(), "direct");
  const auto out = d.download(static_cast<size_t>(m) * n);
  for (uint32_t r = 0; r < m; ++r) {
    for (uint32_t c = 0; c < n; ++c) {
      const float ref = ref_dot(ha, hb, r, c, k);
      require(std::fabs(out[static_cast<size_t>(r) * n + c] - ref) <= 0.002f + 0.002f * std::fabs(ref),
              "direct FP32 result exceeds tolerance");
    }
  }
  args.m = 100;
  require(launch_direct_cute_gemm(args) == KernelStatus::kInvalidArgument,
          "incomplete tiles must be rejected");
}

void probe_case(DeviceSchedulerKind scheduler, uint32_t claim) {
  std::vector<ExpertTile> tiles;
  for (uint32_t i = 0; i < 37; ++i) {
    tiles.push_back({i % 7, i / 7, i % 4, i % 5 == 0 ? 17u : 128u, i % 3 == 0 ? 65u : 128u});
  }
  const uint32_t ctas = 8;
  Dev<ExpertTile> dt(tiles.size());
  Dev<uint32_t> next(1), visits(tiles.size()), cta_tiles(ctas);
  Dev<uint64_t> sums(tiles.size()), cta_work(ctas);
  dt.upload(tiles);
  cuda_ok(cudaMemset(next.p, 0, 4), "memset");
  cuda_ok(cudaMemset(visits.p, 0, tiles.size() * 4), "memset");
  cuda_ok(cudaMemset(cta_tiles.p, 0, ctas * 4), "memset");
  cuda_ok(cudaMemset(cta_work.p, 0, ctas * 8), "memset");
  SchedulerProbeArguments args;
  args.tiles = dt.p; args.tile_count = 37; args.cta_count = ctas; args.claim_size = claim;
  args.work_scale = 2; args.next_tile = next.p; args.tile_visits = visits.p;
  args.tile_checksums = sums.p; args.cta_tile_counts = cta_tiles.p;
  args.cta_valid_elements = cta_work.p;
  const KernelStatus st = launch_scheduler_probe(scheduler, args);
  require(st == KernelStatus::kSuccess, kernel_status_string(st));
  cuda_ok(cudaDeviceSynchronize(), "probe");
  for (uint32_t v : visits.download(tiles.size())) require(v == 1, "tile not visited exactly once");
  const auto per_cta = cta_tiles.download(ctas);
  require(std::accumulate(per_cta.begin(), per_cta.end(), 0u) == 37u, "CTA tile counts do not sum");
  uint64_t want = 0;
  for (const auto& t : tiles) want += valid_output_elements(t);
  const auto work = cta_work.download(ctas);
  require(std::accumulate(work.begin(), work.end(), uint64_t{0}) == want, "CTA work does not sum");
}

}  // namespace

int main() {
  try {
    int device = 0, major = 0, minor = 0;
    cuda_ok(cudaGetDevice(&device), "cudaGetDevice");
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device);
    if (major != 10 || minor != 0) {
      std::printf("SKIP: needs compute capability 10.0 (found %d.%d)\n", major, minor);
      return 0;
    }
    grouped_kat();
    fp8_kat();
    dense_kat<Sm100DenseGemmPlan>(128, 128, 64, 9, 4, 3, 11, 5, "1-CTA dense plan");
    dense_kat<Sm100TwoSmGemmPlan>(256, 128, 64, 7, 3, 5, 13, 6, "CTA-pair dense plan");
    dense_kat<Sm100DenseGemmPlan>(1000, 520, 264, 9, 4, 3, 11, 5, "1-CTA dense plan, ragged");
    dense_kat<Sm100TwoSmGemmPlan>(1000, 520, 264, 7, 3, 5, 13, 6, "CTA-pair dense plan, ragged");
    direct_kat();
    probe_case(DeviceSchedulerKind::kStaticPersistent, 1);
    probe_case(DeviceSchedulerKind::kDynamicQueue, 1);
    probe_case(DeviceSchedulerKind::kDynamicQueue, 4);
    std::printf("drop-in GPU tests passed (%s, %s, %s)\n", sm100_dense_kernel_name(),
                sm100_2sm_kernel_name(), direct_cute_kernel_name());
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "drop-in GPU test failed: %s\n", e.what());
    return 1;
  }
}
