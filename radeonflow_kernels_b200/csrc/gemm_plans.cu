// Tuned-plan table of the FP8 GEMM: exact-shape overrides of the planner's cost model.
//
// The reference picks its kernel instance from a compile-time dispatch table that an offline brute-force
// tuner regenerates (src/gemm/gemm_launcher.cpp:229-247, tuner/gemm_tuner.py:343-385).  Here the kernels are
// shape-generic, so the table only has to hold (tile width, split-K or -1 for stream-K) per shape and can be changed at run
// time: a built-in table measured on B200 for the benchmark shapes, entries registered by the caller
// (rf_fp8_gemm_set_plan), and a text file (rf_fp8_gemm_load_plans, or RF_FP8_GEMM_PLANS at first use)
// written by `python -m radeonflow_kernels_b200.tune`.
#include "../../include/rf_b200.h"
#include "fp8_gemm.h"

#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

namespace rf {

namespace {

struct PlanEntry {
    int block_n;
    int splits;
};

using ShapeKey = std::tuple<int, int, int>;

std::mutex g_mu;
std::map<ShapeKey, PlanEntry> g_plans;
bool g_initialised = false;

// Measured on B200 (148 SMs) by the tuner, rotating operand sets larger than L2; one line per benchmark
// shape of scripts/problems/gemm/task.yml:66-84.  {m, n, k, tile width, split-K}
const int kBuiltin[][5] = {
#include "tuned_plans.inc"
};

bool entry_valid(int m, int n, int k, int block_n, int splits) {
    if (m <= 0 || n <= 0 || k <= 0 || (n % 64) != 0 || (k % 128) != 0) return false;
    if (block_n != 128 && block_n != 256 && block_n != 512) return false;
    return splits == -1 || (splits >= 1 && splits <= k / 128 && splits <= 64);     // -1 = stream-K
}

int load_file_locked(const char* path) {
    FILE* f = fopen(path, "r");
    if (!f) return -1;
    char line[256];
    int loaded = 0;
    bool bad = false;
    while (fgets(line, sizeof line, f)) {
        const char* p = line;
        while (*p == ' ' || *p == '\t') ++p;
        if (*p == '#' || *p == '\n' || *p == '\r' || *p == 0) continue;
        int m, n, k, bn, s;
        if (sscanf(p, "%d %d %d %d %d", &m, &n, &k, &bn, &s) != 5 || !entry_valid(m, n, k, bn, s)) {
            bad = true;
            continue;
        }
        g_plans[ShapeKey(m, n, k)] = PlanEntry{bn, s};
        ++loaded;
    }
    fclose(f);
    return bad ? -2 : loaded;
}

void init_locked() {
    if (g_initialised) return;
    g_initialised = true;
    const char* off = getenv("RF_FP8_GEMM_NO_BUILTIN_PLANS");
    if (!(off && off[0] == '1')) {
        for (const auto& e : kBuiltin)
            if (entry_valid(e[0], e[1], e[2], e[3], e[4])) g_plans[ShapeKey(e[0], e[1], e[2])] = PlanEntry{e[3], e[4]};
    }
    if (const char* path = getenv("RF_FP8_GEMM_PLANS")) {
        if (load_file_locked(path) < 0) fprintf(stderr, "rf_b200: could not read all of RF_FP8_GEMM_PLANS=%s\n", path);
    }
}

}  // namespace

bool tuned_plan_lookup(int m, int n, int k, int* block_n, int* splits) {
    std::lock_guard<std::mutex> lock(g_mu);
    init_locked();
    auto it = g_plans.find(ShapeKey(m, n, k));
    if (it == g_plans.end()) return false;
    *block_n = it->second.block_n;
    *splits = it->second.splits;
    return true;
}

}  // namespace rf

extern "C" {

int rf_fp8_gemm_set_plan(int m, int n, int k, int block_n, int split_k) {
    std::lock_guard<std::mutex> lock(rf::g_mu);
    rf::init_locked();
    if (block_n == 0) {
        rf::g_plans.erase(rf::ShapeKey(m, n, k));
        return RF_OK;
    }
    if (!rf::entry_valid(m, n, k, block_n, split_k)) return RF_ERR_BAD_SHAPE;
    rf::g_plans[rf::ShapeKey(m, n, k)] = rf::PlanEntry{block_n, split_k};
    return RF_OK;
}

int rf_fp8_gemm_load_plans(const char* path) {
    if (!path) return -1;
    std::lock_guard<std::mutex> lock(rf::g_mu);
    rf::init_locked();
    return rf::load_file_locked(path);
}

}  // extern "C"
