// Host-side plan pipeline under AddressSanitizer / UndefinedBehaviorSanitizer (no GPU, no torch):
// load -> validate -> lower (several CTA budgets, with and without multicast) -> check_world for every
// case directory, and load / validate of deliberately broken inputs, which must end in an exception.
//
//   plan_sanitize <dir>
//     <dir>/good/<case>/<rank>.json   one plan per rank, ranks 0..W-1
//     <dir>/bad/<name>.json           texts that must be rejected
// Prints one summary line; exits 0 when every good case went through and every bad one was refused.
#include <dirent.h>
#include <sys/stat.h>

#include <algorithm>
#include <cstdio>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include "common/util.h"
#include "engine/plan.h"

namespace {

std::string slurp(const std::string& path) {
  std::ifstream in(path);
  std::stringstream ss;
  ss << in.rdbuf();
  return ss.str();
}

std::vector<std::string> entries(const std::string& dir) {
  std::vector<std::string> out;
  if (DIR* d = opendir(dir.c_str())) {
    while (dirent* e = readdir(d)) {
      const std::string name = e->d_name;
      if (name != "." && name != "..") out.push_back(name);
    }
    closedir(d);
  }
  std::sort(out.begin(), out.end());
  return out;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc != 2) {
    std::fprintf(stderr, "usage: plan_sanitize <dir>\n");
    return 2;
  }
  const std::string root = argv[1];
  int good = 0, lowered = 0, refused = 0, failures = 0;
  for (const std::string& name : entries(root + "/good")) {
    const std::string dir = root + "/good/" + name;
    const int world = static_cast<int>(entries(dir).size());
    try {
      std::vector<pccl::Plan> plans;
      for (int r = 0; r < world; ++r) plans.push_back(pccl::load_plan(slurp(dir + "/" + std::to_string(r) + ".json")));
      for (int r = 0; r < world; ++r) {
        pccl::PlanLimits limits;
        limits.rank = r; limits.world = world; limits.buffer_elems = int64_t(1) << 32;
        pccl::validate_plan(plans[r], limits);
        for (const uint32_t ctas : {1u, 16u, 128u}) {
          for (const bool multicast : {false, true}) {
            pccl::LowerOptions opt;
            opt.rank = r; opt.world = world; opt.multicast = multicast; opt.total_ctas = ctas;
            opt.closing_barrier = (ctas == 16u);
            const pccl::LoweredProgram lp = pccl::lower_plan(plans[r], opt);
            if (lp.chains.empty() && !plans[r].ops.empty()) throw pccl::Error("lowering produced no chain");
            ++lowered;
          }
        }
      }
      const pccl::WorldReport report = pccl::check_world(plans);
      if (report.deadlock || report.leftover_signals != 0) throw pccl::Error("protocol check: " + report.detail);
      ++good;
    } catch (const std::exception& e) {
      std::fprintf(stderr, "FAILED good case %s: %s\n", name.c_str(), e.what());
      ++failures;
    }
  }
  for (const std::string& name : entries(root + "/bad")) {
    try {
      const pccl::Plan plan = pccl::load_plan(slurp(root + "/bad/" + name));
      pccl::PlanLimits limits;
      limits.rank = 0; limits.world = 2; limits.buffer_elems = 1 << 20;
      pccl::validate_plan(plan, limits);
      std::fprintf(stderr, "FAILED bad case %s was accepted\n", name.c_str());
      ++failures;
    } catch (const std::exception&) {
      ++refused;
    }
  }
  std::printf("PLAN_SANITIZE good=%d lowered=%d refused=%d failures=%d\n", good, lowered, refused, failures);
  return failures == 0 ? 0 : 1;
}
