// Test driver for the TinyTorch binding of libtt_attn.so (tinytorch_b200/shim/TinyTorchFusedAttention.h).
//
// It is compiled against a CUDA-enabled build of the unmodified reference sources and calls
// function::sdpAttentionFused the way the one-line patch of the reference's call site
// (src/Function/FuncNNLayer.h:298-302) would: Function<>::apply (src/Tensor/Function.h:106-144),
// the dispatch table (src/Tensor/Dispatch.h:110-142), AutogradMeta::addGrad
// (src/Tensor/AutogradMeta.cpp:29-43).  Tensors travel as raw float32 files; the pytest side
// (tests/test_shim_gpu.py) makes the inputs and checks the outputs.
//
//   shim_driver fwd    <dtype> <N> <Hq> <Hkv> <L> <S> <D> <causal> <impl> <chunk> <offset> q k v out
//       impl = fused : function::sdpAttentionFused on the whole [N,Hq,L,D] problem
//       impl = ref   : the reference's own function::sdpAttention (its CUDA composition), <chunk>
//                      batch entries per call (its large-row softmax launch needs N*Hq*L <= 65535 per call,
//                      src/Operation/OpNNLayerCuda.cuh:375)
//       offset       : q is made a view that starts <offset> elements into a larger storage
//   shim_driver fwdbwd <dtype> <N> <Hq> <Hkv> <L> <S> <D> <causal> <reps> <needq> <needk> <needv> q k v do out dq dk dv
//       <reps> times: y = sdpAttentionFused(q, k, v); y.backward(dO)   (gradients accumulate on the leaves)
//   shim_driver decode <dtype> <N> <Hq> <Hkv> <S> <D> <impl> lens q k v out
//       impl = fused : op::sdpAttentionDecode through the dispatch table (one query per sequence against a cache
//                      of capacity S with per-sequence lengths, a float32 file of N values)
//       impl = ref   : what a TinyTorch caller writes without it: function::sdpAttention with a Bool mask
//                      [N,1,1,S] built from the lengths (K / V repeated for grouped-query shapes)
//   shim_driver fusedops <dtype> <rows> <dim> <nout>
//       the block operators either side of attention (tinytorch_b200/shim/TinyTorchFusedOps.h): op::siluMul,
//       op::fusedAddRmsNorm and function::linear's product are first computed by the reference's own CUDA
//       implementations, then registerFusedOpsB200() replaces the dispatch-table entries and the same calls run
//       again; prints the largest absolute differences (silu= rms_input= rms_residual= linear=)
// Each run prints one line: fused_calls=<n> ms=<device time of the timed call(s)>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "TinyTorch.h"
#include "TinyTorchFusedAttention.h"
#include "TinyTorchFusedOps.h"
#include "Utils/RandomGenerator.h"

using namespace tinytorch;

static std::vector<float> readf(const char* path, size_t n) {
  std::vector<float> v(n);
  FILE* f = fopen(path, "rb");
  if (!f || fread(v.data(), 4, n, f) != n) {
    fprintf(stderr, "cannot read %zu floats from %s\n", n, path);
    exit(2);
  }
  fclose(f);
  return v;
}

static void writef(const char* path, const Tensor& t) {
  std::vector<float> v = t.to(DType::Float32).to(Device(DeviceType::CPU)).toList<float>();
  FILE* f = fopen(path, "wb");
  if (!f || fwrite(v.data(), 4, v.size(), f) != v.size()) {
    fprintf(stderr, "cannot write %s\n", path);
    exit(2);
  }
  fclose(f);
}

static float maxAbsDiff(const Tensor& a, const Tensor& b) {
  std::vector<float> x = a.to(DType::Float32).to(Device(DeviceType::CPU)).toList<float>();
  std::vector<float> y = b.to(DType::Float32).to(Device(DeviceType::CPU)).toList<float>();
  float m = x.size() == y.size() ? 0.f : 1e30f;
  for (size_t i = 0; i < x.size() && i < y.size(); i++) {
    const float d = std::fabs(x[i] - y[i]);
    if (!(d <= m)) m = d;  // NaN propagates
  }
  return m;
}

static Tensor copyOf(const Tensor& t) {
  Tensor c(t.shape(), t.options().noGrad());
  c.copy_(t);
  return c;
}

static DType parseDType(const char* s) {
  if (!strcmp(s, "f32")) return DType::Float32;
  if (!strcmp(s, "f16")) return DType::Float16;
  if (!strcmp(s, "bf16")) return DType::BFloat16;
  fprintf(stderr, "bad dtype %s\n", s);
  exit(2);
}

static Tensor upload(const char* path, const std::vector<int64_t>& shape, DType dt, bool requiresGrad) {
  size_t n = 1;
  for (auto d : shape) n *= static_cast<size_t>(d);
  Tensor host(readf(path, n), IntArrayView(shape));
  Tensor dev = host.to(dt, Device(DeviceType::CUDA, 0));
  if (requiresGrad) dev.setRequiresGrad(true);
  return dev;
}

// the same values as `t`, as a view that starts `offset` elements into a larger storage
static Tensor offsetView(const Tensor& t, int64_t offset) {
  Tensor big({t.numel() + offset}, t.options().noGrad());
  Tensor view(t.shape(), t.options().noGrad(), big.storage(), offset);
  view.copy_(t);
  return view;
}

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  const std::string cmd = argv[1];
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  float ms = 0.f;
  if (cmd == "fwd" && argc == 17) {
    const DType dt = parseDType(argv[2]);
    const int64_t N = atoll(argv[3]), Hq = atoll(argv[4]), Hkv = atoll(argv[5]), L = atoll(argv[6]), S = atoll(argv[7]),
                  D = atoll(argv[8]);
    const bool causal = atoi(argv[9]) != 0;
    const std::string impl = argv[10];
    const int64_t chunk = atoll(argv[11]), offset = atoll(argv[12]);
    NoGradGuard guard;
    Tensor q = upload(argv[13], {N, Hq, L, D}, dt, false);
    Tensor k = upload(argv[14], {N, Hkv, S, D}, dt, false);
    Tensor v = upload(argv[15], {N, Hkv, S, D}, dt, false);
    if (offset > 0) q = offsetView(q, offset);
    Tensor out;
    auto stream = cuda::getCurrentCUDAStream(0).stream();
    if (impl == "fused") {
      out = function::sdpAttentionFused(q, k, v, causal);  // warm-up (first call loads the kernels)
      cudaEventRecord(e0, stream);
      out = function::sdpAttentionFused(q, k, v, causal);
      cudaEventRecord(e1, stream);
    } else {
      // the reference's own composition; chunks of whole batch entries are independent
      out = Tensor({N, Hq, L, D}, q.options().noGrad());
      for (int pass = 0; pass < 2; pass++) {  // pass 0 warms up
        if (pass == 1) cudaEventRecord(e0, stream);
        for (int64_t b0 = 0; b0 < N; b0 += chunk) {
          const int64_t n = std::min(chunk, N - b0);
          Tensor o = function::sdpAttention(q.narrow(0, b0, n), k.narrow(0, b0, n), v.narrow(0, b0, n), causal);
          Tensor dst({n, Hq, L, D}, out.options(), out.storage(), b0 * Hq * L * D);
          dst.copy_(o);
        }
        if (pass == 1) cudaEventRecord(e1, stream);
      }
    }
    cudaEventSynchronize(e1);
    cudaEventElapsedTime(&ms, e0, e1);
    writef(argv[16], out);
  } else if (cmd == "fwdbwd" && argc == 22) {
    const DType dt = parseDType(argv[2]);
    const int64_t N = atoll(argv[3]), Hq = atoll(argv[4]), Hkv = atoll(argv[5]), L = atoll(argv[6]), S = atoll(argv[7]),
                  D = atoll(argv[8]);
    const bool causal = atoi(argv[9]) != 0;
    const int reps = atoi(argv[10]);
    const bool nq = atoi(argv[11]) != 0, nk = atoi(argv[12]) != 0, nv = atoi(argv[13]) != 0;
    Tensor q = upload(argv[14], {N, Hq, L, D}, dt, nq);
    Tensor k = upload(argv[15], {N, Hkv, S, D}, dt, nk);
    Tensor v = upload(argv[16], {N, Hkv, S, D}, dt, nv);
    Tensor dO = upload(argv[17], {N, Hq, L, D}, dt, false);
    Tensor y;
    auto stream = cuda::getCurrentCUDAStream(0).stream();
    cudaEventRecord(e0, stream);
    for (int r = 0; r < reps; r++) {
      y = function::sdpAttentionFused(q, k, v, causal);
      y.backward(dO);
    }
    cudaEventRecord(e1, stream);
    cudaEventSynchronize(e1);
    cudaEventElapsedTime(&ms, e0, e1);
    writef(argv[18], y);
    const Tensor* leaves[3] = {&q, &k, &v};
    const bool need[3] = {nq, nk, nv};
    for (int i = 0; i < 3; i++) {
      // a leaf that does not require a gradient must not have received one
      if (need[i]) {
        writef(argv[19 + i], leaves[i]->grad());
      } else {
        if (leaves[i]->requiresGrad()) return 3;
        writef(argv[19 + i], Tensor::zeros(leaves[i]->shape()));
      }
    }
  } else if (cmd == "fusedops" && argc == 6) {
    const DType dt = parseDType(argv[2]);
    const int64_t rows = atoll(argv[3]), dim = atoll(argv[4]), nout = atoll(argv[5]);
    NoGradGuard guard;
    const Device dev(DeviceType::CUDA, 0);
    manualSeed(1234);
    Tensor x = Tensor::randn({rows, 2 * dim}, options::device(dev)).to(dt);
    Tensor h = Tensor::randn({rows, dim}, options::device(dev)).to(dt);
    Tensor res = Tensor::randn({rows, dim}, options::device(dev)).to(dt);
    Tensor w = Tensor::randn({dim}, options::device(dev)).to(dt);
    Tensor lw = (Tensor::randn({nout, dim}, options::device(dev)) * 0.05f).to(dt);
    Tensor lb = Tensor::randn({nout}, options::device(dev)).to(dt);
    // the reference's own CUDA implementations
    Tensor silu0 = op::siluMul(x);
    Tensor h0 = copyOf(h), res0 = copyOf(res);
    op::fusedAddRmsNorm(h0, res0, w, 1e-5f);
    Tensor lin0 = op::matmul(h, lw, false, true, lb);
    // the B200 kernels behind the same dispatch-table entries
    op::registerFusedOpsB200();
    Tensor silu1 = op::siluMul(x);
    Tensor h1 = copyOf(h), res1 = copyOf(res);
    op::fusedAddRmsNorm(h1, res1, w, 1e-5f);
    Tensor lin1 = op::linearOpB200(h, lw, lb);
    // (linearOpB200 declines what its kernel does not cover, fp32 for one, by returning an undefined tensor: -1)
    printf("silu=%g rms_input=%g rms_residual=%g linear=%g ", maxAbsDiff(silu0, silu1), maxAbsDiff(h0, h1),
           maxAbsDiff(res0, res1), lin1.defined() ? maxAbsDiff(lin0, lin1) : -1.f);
  } else if (cmd == "decode" && argc == 14) {
    const DType dt = parseDType(argv[2]);
    const int64_t N = atoll(argv[3]), Hq = atoll(argv[4]), Hkv = atoll(argv[5]), S = atoll(argv[6]), D = atoll(argv[7]);
    const std::string impl = argv[8];
    NoGradGuard guard;
    std::vector<float> lensf = readf(argv[9], static_cast<size_t>(N));
    Tensor q = upload(argv[10], {N, Hq, 1, D}, dt, false);
    Tensor k = upload(argv[11], {N, Hkv, S, D}, dt, false);
    Tensor v = upload(argv[12], {N, Hkv, S, D}, dt, false);
    auto stream = cuda::getCurrentCUDAStream(0).stream();
    Tensor out;
    if (impl == "fused") {
      std::vector<int32_t> li(lensf.begin(), lensf.end());
      Tensor lens = Tensor(li, IntArrayView({N}), options::dtype(DType::Int32)).to(Device(DeviceType::CUDA, 0));
      const float scale = 1.f / std::sqrt(static_cast<float>(D));
      out = op::sdpAttentionDecode(q, k, v, lens, scale);  // warm-up
      cudaEventRecord(e0, stream);
      out = op::sdpAttentionDecode(q, k, v, lens, scale);
      cudaEventRecord(e1, stream);
    } else {
      std::vector<uint8_t> m(static_cast<size_t>(N * S));
      for (int64_t b = 0; b < N; b++)
        for (int64_t j = 0; j < S; j++) m[b * S + j] = j < static_cast<int64_t>(lensf[b]) ? 1 : 0;
      Tensor mask = Tensor(m, IntArrayView({N, 1, 1, S}), options::dtype(DType::Bool)).to(Device(DeviceType::CUDA, 0));
      const int64_t g = Hq / Hkv;
      Tensor kk = g > 1 ? function::repeatInterleave(k, g, 1) : k;
      Tensor vv = g > 1 ? function::repeatInterleave(v, g, 1) : v;
      out = function::sdpAttention(q, kk, vv, false, mask);  // warm-up
      cudaEventRecord(e0, stream);
      out = function::sdpAttention(q, kk, vv, false, mask);
      cudaEventRecord(e1, stream);
    }
    cudaEventSynchronize(e1);
    cudaEventElapsedTime(&ms, e0, e1);
    writef(argv[13], out);
  } else {
    fprintf(stderr, "usage: see the header of tests/cxx/shim_driver.cpp\n");
    return 2;
  }
  printf("fused_calls=%ld ms=%.4f\n", fused_detail::fusedCalls().load(), ms);
  return 0;
}
