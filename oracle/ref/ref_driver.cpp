// Runs the reference's rwkv::Model on a `.fr` file and dumps the logits of every step as raw float32.
// TEST INFRASTRUCTURE ONLY.  usage: fr_ref_run <model.fr> <strategy> <out.bin> [--seq] id id id ...
// Without --seq every id goes through Model::Run(int) (model.cpp:205); with --seq all ids go through
// Model::Run(vector) once (model.cpp:188-203) and only the last logits are written.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <vector>

#include <model.h>

int main(int argc, char **argv) {
  if (argc < 5) {
    std::fprintf(stderr, "usage: %s model.fr strategy out.bin [--seq] ids...\n", argv[0]);
    return 2;
  }
  try {
    rwkv::Model model(argv[1], argv[2]);
    std::ofstream out(argv[3], std::ios::binary);
    bool seq = false;
    std::vector<int> ids;
    for (int i = 4; i < argc; ++i) {
      if (!std::strcmp(argv[i], "--seq")) seq = true;
      else ids.push_back(std::atoi(argv[i]));
    }
    auto dump = [&](const rwkv::Tensor &t) {
      out.write(reinterpret_cast<const char *>(t.data_ptr<float>()), t.numel() * sizeof(float));
    };
    if (seq) dump(model.Run(ids));
    else for (int id : ids) dump(model.Run(id));
    if (std::getenv("FR_REF_STATE")) model.SaveStateFile(std::getenv("FR_REF_STATE"));
  } catch (const std::exception &e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  return 0;
}
