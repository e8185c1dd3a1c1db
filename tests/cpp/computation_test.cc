// C++ use of the library through include/cinn_b200_frontend.hpp, written the way the reference's own
// cinn/frontend/computation_test.cc:74-103 is: build a program with NetBuilder, compile it, feed inputs, run, check.
//   argv[1] = "plan": no GPU is touched (fusion + kernel matching only), prints the groups
//   argv[1] = "run" : executes on device 0 and checks A + (A + B) == 2A + B and the transposed, reduced results
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "cinn_b200_frontend.hpp"

using cinn_b200::frontend::CinnComputation;
using cinn_b200::frontend::NetBuilder;

int main(int argc, char** argv) {
  const bool run = argc > 1 && !strcmp(argv[1], "run");
  const int M = 32, N = 24;
  try {
    {
      // program passes: cast(cast(cast(x, int32), int64), float32) collapses to x (cast_collapsing_test.cc:90-109)
      NetBuilder pb("pass_builder");
      auto x   = pb.CreateInput("float32", {4, 5, 3}, "X");
      auto o   = pb.Cast(pb.Cast(pb.Cast(x, "int32"), "int64"), "float32");
      auto sum = pb.Add(o, o);
      pb.ApplyPasses({sum}, {"CastCollapsing"});
      if (pb.ProgramText().find("cast") != std::string::npos || pb.ProgramText().find("= X, X") == std::string::npos) {
        printf("FAILED: CastCollapsing left %s\n", pb.ProgramText().c_str());
        return 1;
      }
    }
    {
      // CompileOptions::use_decomposer: gelu and the max-subtracted softmax as instructions, decomposed at compile time
      NetBuilder db("decomposed");
      auto x = db.CreateInput("float32", {64, 4096}, "X");
      auto g = db.Softmax(db.Gelu(x), {-1}, "safe");
      CinnComputation::CompileOptions options = CinnComputation::DefaultCompileOptions();
      options.use_decomposer = true;
      auto comp = CinnComputation::BuildAndCompile(-1, db, options, {g});
      bool safe = false;
      for (auto& p : comp->GroupPatterns()) safe = safe || p.find("softmax_safe_row") != std::string::npos;
      if (!safe || db.ProgramText().find("gelu") != std::string::npos) {
        printf("FAILED: the decomposer left %s\n", db.ProgramText().c_str());
        return 1;
      }
    }
    NetBuilder builder("net_builder");
    auto a   = builder.CreateInput("float32", {M, N}, "A");
    auto b   = builder.CreateInput("float32", {M, N}, "B");
    auto c   = builder.Add(a, b);
    auto d   = builder.Add(a, c);                       // 2A + B
    auto t   = builder.Transpose(builder.Relu(d), {1, 0});
    auto s   = builder.ReduceSum(builder.Multiply(d, builder.Identity(d)), {1});
    auto cmp = builder.GreaterThan(d, builder.FillConstant({M, N}, 0.0f));
    auto computation = CinnComputation::BuildAndCompile(run ? 0 : -1, builder, {d, t, s, cmp});
    for (auto& g : computation->GroupPatterns()) printf("group: %s\n", g.c_str());
    // the ahead-of-time path: export, load, same groups
    auto loaded = CinnComputation::Load(computation->Export(), run ? 0 : -1);
    if (loaded->GroupPatterns().size() != computation->GroupPatterns().size()) {
      printf("FAILED: the loaded program has a different number of groups\n");
      return 1;
    }
    if (computation->GetInputTensors().size() != 2 || computation->GetOutputTensors().size() != 3 ||
        computation->GetTensor("A").shape != std::vector<int64_t>{M, N} || computation->GetTensor(cmp.id).dtype != "bool") {
      printf("FAILED: inputs / outputs of the computation are not what the program declares\n");
      return 1;
    }
    if (!run) {
      printf("PLANNED\n");
      return 0;
    }
    std::mt19937 rng(7);
    std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
    std::vector<float> ha(M * N), hb(M * N), hd(M * N), ht(M * N), hs(M);
    std::vector<unsigned char> hc(M * N);
    for (auto& v : ha) v = dist(rng);
    for (auto& v : hb) v = dist(rng);
    for (auto* comp : {computation.get(), loaded.get()}) {
      comp->SetTensorData("A", ha.data(), ha.size() * 4);
      comp->SetTensorData("B", hb.data(), hb.size() * 4);
      comp->Execute();
      comp->GetTensorData(d.id, hd.data(), hd.size() * 4);
      comp->GetTensorData(t.id, ht.data(), ht.size() * 4);
      comp->GetTensorData(s.id, hs.data(), hs.size() * 4);
      comp->GetTensorData(cmp.id, hc.data(), hc.size());
      for (int i = 0; i < M; ++i) {
        double row = 0.0;
        for (int j = 0; j < N; ++j) {
          const float want = ha[i * N + j] + (ha[i * N + j] + hb[i * N + j]);
          if (hd[i * N + j] != want || ht[j * M + i] != (want > 0.0f ? want : 0.0f) || hc[i * N + j] != (want > 0.0f)) {
            printf("FAILED at (%d, %d): %g vs %g\n", i, j, hd[i * N + j], want);
            return 1;
          }
          row += (double)want * want;
        }
        if (std::fabs(hs[i] - row) > 1e-5 * row + 1e-6) {
          printf("FAILED: row sum %d: %g vs %g\n", i, hs[i], row);
          return 1;
        }
      }
    }
    printf("average run: %.2f us launch by launch, %.2f us from one CUDA graph\n", computation->ExecuteTest(200) * 1e3,
           computation->ExecuteTest(200, true) * 1e3);
    printf("PASSED\n");
    return 0;
  } catch (const std::exception& e) {
    printf("FAILED: %s\n", e.what());
    return 1;
  }
}
