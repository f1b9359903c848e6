// Runs the reference's rwkv::Model on a `.fr` file and dumps the logits of every step as raw float32.
// usage: fr_run <model.fr> <strategy> <out.bin> [--seq] id id id ...
// Without --seq every id goes through Model::Run(int) (model.cpp:205); with --seq all ids go through
// Model::Run(vector) once (model.cpp:188-203) and only the last logits are written.
// --bench N: after the ids, N greedy tokens through Model::Run(int) (host argmax, as bench_model.cpp:5-10 times
// Run + the copy to the host) are timed with the wall clock; prints "ms_per_token <x>".
// --time-seq N (with --seq): the prompt is run N more times from reset states, each Run(vector) (which ends with the
// copy of the logits to the host) timed with the wall clock; prints "ms_per_prompt <fastest>".
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <vector>

#include <kernels/kernels.h>
#include <model.h>
#include <sampler.h>

// --ops-test: the body of the reference's tests/test_ops.cpp:9-16 on the registered CUDA operators: fill_(1) then
// scalar_div_(2) must leave 0.5 in every element.  Prints "ops_test ok".
static int ops_test() {
  try {
    for (rwkv::DType dt : {rwkv::DType::kFloat16, rwkv::DType::kFloat32}) {
      rwkv::Tensor x = rwkv::Tensor::Empty({2, 3}, dt, rwkv::Device::kCUDA);
      rwkv::fill_(x, 1.f);
      rwkv::scalar_div_(x, 2.f);
      rwkv::Tensor y = rwkv::cast_dtype(x, rwkv::DType::kFloat32);
      rwkv::Tensor h = rwkv::Copy(y, rwkv::Device::kCPU);
      for (int i = 0; i < 6; ++i)
        if (h.data_ptr<float>()[i] != 0.5f) { std::fprintf(stderr, "ops_test: element %d is %g\n", i, h.data_ptr<float>()[i]); return 1; }
    }
  } catch (const std::exception &e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  std::printf("ops_test ok\n");
  return 0;
}

// --sample logits.bin V rows temperature top_k top_p seed draws: the reference's own Sampler (sampler.cpp:38-101, with its
// CPU softmax) on `rows` rows of V fp32 logits; for every row the generator is seeded with `seed` and `draws` tokens
// are drawn from the same logits.  Prints one line "sample <row> <id> <id> ..." per row.
static int sample_mode(int argc, char **argv) {
  if (argc < 10) { std::fprintf(stderr, "usage: --sample logits.bin V rows temperature top_k top_p seed draws\n"); return 2; }
  try {
    const int V = std::atoi(argv[3]), rows = std::atoi(argv[4]), top_k = std::atoi(argv[6]), seed = std::atoi(argv[8]), draws = std::atoi(argv[9]);
    const float temperature = (float)std::atof(argv[5]), top_p = (float)std::atof(argv[7]);
    std::ifstream in(argv[2], std::ios::binary);
    if (!in.good()) { std::fprintf(stderr, "error: cannot open %s\n", argv[2]); return 1; }
    rwkv::Sampler sampler;
    for (int r = 0; r < rows; ++r) {
      rwkv::Tensor logits = rwkv::Tensor::Empty({V}, rwkv::DType::kFloat32, rwkv::Device::kCPU);
      in.read(reinterpret_cast<char *>(logits.data_ptr<float>()), (std::streamsize)V * 4);
      sampler.set_seed(seed);
      std::printf("sample %d", r);
      for (int d = 0; d < draws; ++d) std::printf(" %d", sampler.Sample(logits, temperature, top_k, top_p));
      std::printf("\n");
    }
  } catch (const std::exception &e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  return 0;
}

int main(int argc, char **argv) {
  if (argc >= 2 && !std::strcmp(argv[1], "--ops-test")) return ops_test();
  if (argc >= 2 && !std::strcmp(argv[1], "--sample")) return sample_mode(argc, argv);
  if (argc < 5) {
    std::fprintf(stderr, "usage: %s model.fr strategy out.bin [--seq] ids...\n", argv[0]);
    return 2;
  }
  try {
    rwkv::Model model(argv[1], argv[2]);
    std::ofstream out(argv[3], std::ios::binary);
    bool seq = false;
    int bench = 0, time_seq = 0;
    std::vector<int> ids;
    for (int i = 4; i < argc; ++i) {
      if (!std::strcmp(argv[i], "--seq")) seq = true;
      else if (!std::strcmp(argv[i], "--bench") && i + 1 < argc) bench = std::atoi(argv[++i]);
      else if (!std::strcmp(argv[i], "--time-seq") && i + 1 < argc) time_seq = std::atoi(argv[++i]);
      else ids.push_back(std::atoi(argv[i]));
    }
    auto dump = [&](const rwkv::Tensor &t) {
      out.write(reinterpret_cast<const char *>(t.data_ptr<float>()), t.numel() * sizeof(float));
    };
    if (seq) dump(model.Run(ids));
    else for (int id : ids) dump(model.Run(id));
    if (seq && time_seq > 0) {
      double best = 1e30;
      for (int i = 0; i < time_seq; ++i) {
        model.ResetStates();
        auto t0 = std::chrono::steady_clock::now();
        rwkv::Tensor t = model.Run(ids);
        auto t1 = std::chrono::steady_clock::now();
        best = std::min(best, std::chrono::duration<double, std::milli>(t1 - t0).count());
      }
      std::printf("ms_per_prompt %.6f\n", best);
    }
    if (bench > 0) {
      auto greedy = [&](int id) {
        rwkv::Tensor t = model.Run(id);
        const float *p = t.data_ptr<float>();
        int best = 0;
        for (long i = 1; i < t.numel(); ++i) if (p[i] > p[best]) best = (int)i;
        return best;
      };
      int id = ids.empty() ? 0 : ids.back();
      for (int i = 0; i < 8; ++i) id = greedy(id);   // warm-up
      auto t0 = std::chrono::steady_clock::now();
      for (int i = 0; i < bench; ++i) id = greedy(id);
      auto t1 = std::chrono::steady_clock::now();
      std::printf("ms_per_token %.6f\n", std::chrono::duration<double, std::milli>(t1 - t0).count() / bench);
    }
    if (std::getenv("FR_REF_STATE")) model.SaveStateFile(std::getenv("FR_REF_STATE"));
    if (const char *sf = std::getenv("FR_STATE_ROUNDTRIP")) {
      // the sequence of the reference's tests/test_model.cpp:35-51: save the state, run a token, load the state back,
      // run the same token again -- both logits are written after the ids' own
      const int id = ids.empty() ? 0 : ids.front();
      model.SaveStateFile(sf);
      dump(model.Run(id));
      model.LoadStateFile(sf);
      dump(model.Run(id));
    }
  } catch (const std::exception &e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  return 0;
}
