// Stage-level checker of the MoE layer, in C++, for librf_b200.so.
//
// The counterpart of the reference's case plug-in tests/moe/moe_topk_test.cpp (loaded by tests/checker/checker.cpp):
// it builds a seeded layer, calls `run_topk` through dlopen/dlsym exactly as the reference's checker does
// (tests/moe/moe_topk_test.cpp:400-420), recomputes every stage on the CPU and compares the named
// intermediate tensors one by one (the reference's list, :599-611, plus the three it leaves commented out:
// seq_experts_index, permuted_rows, rev_permuted_rows - integer stages are exact here), then prints the
// twelve PerfMetrics entries (src/moe/moe.cpp:350-364).  No libtorch: the CPU side is plain C++ with OpenMP.
//
//   rf_moe_stage_check [--lib PATH] [-c CASE] [-l] [--full] [--dump DIR]
//     -l       list the cases and exit (needs no GPU)
//     --dump DIR  with -c N: write the case's inputs and CPU stage tensors to DIR and exit (needs no GPU)
//     -c N     run only case N
//     --full   the reference's own parameter sets (d_hidden 7168, d_expert 2048; minutes of CPU time)
//   exit code = number of failing stage tensors (0 = all cases passed), 100 = set-up error.
//
// Build: nvcc -O2 -std=c++17 -Xcompiler -fopenmp,-ffp-contract=off -o rf_moe_stage_check rf_moe_stage_check.cu -ldl
#include "../../include/rf_b200.h"

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <string>
#include <vector>

namespace {

// ------------------------------------------------------------------------------------ cases --
// Reference parameter sets: tests/moe/moe_topk_test.cpp:15-62.  The default list keeps their token /
// expert structure with a smaller hidden size so that the CPU recomputation takes seconds.
const InputParams kFullCases[] = {
    {1, 512, 7168, 2048, 4, 4, 1, 9371},  {1, 512, 7168, 2048, 8, 4, 1, 2291},  {2, 512, 7168, 2048, 8, 4, 1, 2291},
    {1, 8192, 7168, 2048, 8, 4, 1, 81934}, {1, 2048, 7168, 2048, 32, 4, 1, 9371}, {1, 8192, 7168, 2048, 32, 4, 1, 1212},
};
const InputParams kSmallCases[] = {
    {1, 512, 1024, 512, 4, 4, 1, 9371},  {1, 512, 1024, 512, 8, 4, 1, 2291},   {2, 512, 1024, 512, 8, 4, 1, 2291},
    {1, 1000, 1024, 512, 32, 4, 1, 9371}, {1, 333, 512, 256, 64, 6, 1, 1212},  {1, 777, 512, 256, 256, 8, 2, 77},
};

// ------------------------------------------------------------------------------ fp16 helpers --
inline uint16_t f2h(float x) {
    const __half h = __float2half_rn(x);
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}
inline float h2f(uint16_t u) {
    __half h;
    memcpy(&h, &u, 2);
    return __half2float(h);
}

// ------------------------------------------------------------------------------------- RNG --
struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 0x1234567ull) {}
    uint64_t next() {
        uint64_t z = (s += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    double uniform() { return ((next() >> 11) + 0.5) * (1.0 / 9007199254740992.0); }
    float normal() {
        const double u1 = uniform(), u2 = uniform();
        return (float)(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
    }
};

std::vector<uint16_t> randn_fp16(Rng& rng, size_t n, float scale) {
    std::vector<uint16_t> v(n);
    for (size_t i = 0; i < n; ++i) v[i] = f2h(rng.normal() * scale);
    return v;
}

// ------------------------------------------------------------------------- CPU restatement --
// out[r, :] = fp16(x[r, :] . w) with w [k, n] row-major, fp32 accumulation.
void linear_fp16(const uint16_t* x, size_t rows, int k, const uint16_t* w, int n, uint16_t* out) {
    std::vector<float> wf((size_t)k * n);
    for (size_t i = 0; i < wf.size(); ++i) wf[i] = h2f(w[i]);
#pragma omp parallel
    {
        std::vector<float> acc(n);
#pragma omp for schedule(dynamic, 8)
        for (long long r = 0; r < (long long)rows; ++r) {
            std::fill(acc.begin(), acc.end(), 0.f);
            const uint16_t* xr = x + (size_t)r * k;
            for (int kk = 0; kk < k; ++kk) {
                const float xv = h2f(xr[kk]);
                const float* wr = wf.data() + (size_t)kk * n;
                for (int j = 0; j < n; ++j) acc[j] += xv * wr[j];
            }
            for (int j = 0; j < n; ++j) out[(size_t)r * n + j] = f2h(acc[j]);
        }
    }
}

// fp16(SiLU(fp16 g)) * fp16 u, rounded to fp16: the rounding points of scripts/problems/moe/reference.py:23-24.
void swiglu_fp16(const uint16_t* g, const uint16_t* u, size_t n, uint16_t* out) {
#pragma omp parallel for
    for (long long i = 0; i < (long long)n; ++i) {
        const float gv = h2f(g[i]);
        const uint16_t s = f2h(gv / (1.0f + std::exp(-gv)));
        out[i] = f2h(h2f(s) * h2f(u[i]));
    }
}

// exp(x), x <= 0: the kernel's fixed fp32 sequence (no FMA contraction: compiled with -ffp-contract=off).
float det_exp(float x) {
    x = std::max(x, -80.0f);
    const float t = x * 1.4426950408889634f;
    const float n = std::nearbyint(t);
    const float f = t - n;
    float p = 1.5252733804059840e-05f;
    const float c[7] = {0.0001540353039338161f, 0.0013333558146428443f, 0.009618129107628477f, 0.05550410866482158f,
                        0.2402265069591007f,    0.6931471805599453f,    1.0f};
    for (float ci : c) {
        p = p * f;
        p = p + ci;
    }
    return std::ldexp(p, (int)n);
}

struct Stages {
    std::vector<int> seq_experts_index, source_rows, permuted_experts, permuted_rows, first_token_offset,
        rev_permuted_rows;
    std::vector<uint16_t> seq_experts_softmax, expanded_seq_input, expanded_seq_softmax, expanded_fc1_output,
        expanded_fc2_output, shared_fc1_output, shared_fc2_output, final_output;
};

// src/moe/moe_topk_kernel.cpp:65-148 - fp16 row max, fp32 exp and sum (32-lane layout, xor butterfly),
// prob = fp16(e * (1 / sum)), k rounds of arg-max with the lowest index winning ties.
void route(const std::vector<uint16_t>& logits, int T, int E, int K, Stages& s) {
    s.seq_experts_index.assign((size_t)T * K, 0);
    s.seq_experts_softmax.assign((size_t)T * K, 0);
    s.source_rows.assign((size_t)T * K, 0);
    const int v = std::max(E / 32, 1);
#pragma omp parallel for
    for (int t = 0; t < T; ++t) {
        std::vector<float> e(E);
        float mx = -INFINITY;
        for (int j = 0; j < E; ++j) mx = std::max(mx, h2f(logits[(size_t)t * E + j]));
        for (int j = 0; j < E; ++j) e[j] = det_exp(h2f(logits[(size_t)t * E + j]) - mx);
        float lanes[32] = {};
        for (int l = 0; l < 32 && l * v < E; ++l) {
            float a = e[l * v];
            for (int j = 1; j < v; ++j) a = a + e[l * v + j];
            lanes[l] = a;
        }
        for (int stride = 16; stride >= 1; stride >>= 1) {
            float nxt[32];
            for (int l = 0; l < 32; ++l) nxt[l] = lanes[l] + lanes[l ^ stride];
            memcpy(lanes, nxt, sizeof lanes);
        }
        const float r = 1.0f / lanes[0];
        std::vector<uint16_t> p16(E);
        std::vector<float> p(E);
        for (int j = 0; j < E; ++j) {
            p16[j] = f2h(e[j] * r);
            p[j] = h2f(p16[j]);
        }
        for (int i = 0; i < K; ++i) {
            int best = 0;
            for (int j = 1; j < E; ++j)
                if (p[j] > p[best]) best = j;
            s.seq_experts_index[(size_t)t * K + i] = best;
            s.seq_experts_softmax[(size_t)t * K + i] = p16[best];
            s.source_rows[(size_t)t * K + i] = i * T + t;
            p[best] = -INFINITY;
        }
    }
}

struct Layer {
    InputParams q;
    int T, d, f, fs, E, K;
    std::vector<uint16_t> x, logits, shared_gate, shared_up, shared_down;
    std::vector<std::vector<uint16_t>> gate, up, down;      // per expert, [in, out] row-major
};

// Weight scales of the reference generator (tests/moe/moe_topk_test.cpp:426-440: gate / up by 1/sqrt(d_expert),
// down by 1/sqrt(d_hidden)); the logits are x . router^T rounded to fp16, the input `run_topk` expects.
Layer make_layer(const InputParams& q) {
    Layer L;
    L.q = q;
    L.T = q.batch_size * q.seq_len;
    L.d = q.d_hidden;
    L.f = q.d_expert;
    L.fs = q.d_expert * q.n_shared_experts;
    L.E = q.n_routed_experts;
    L.K = q.n_experts_per_token;
    Rng rng((uint64_t)q.seed);
    L.x = randn_fp16(rng, (size_t)L.T * L.d, 1.0f);
    std::vector<uint16_t> router = randn_fp16(rng, (size_t)L.E * L.d, 1.0f / std::sqrt((float)L.d));
    for (int e = 0; e < L.E; ++e) {
        L.gate.push_back(randn_fp16(rng, (size_t)L.d * L.f, 1.0f / std::sqrt((float)L.f)));
        L.up.push_back(randn_fp16(rng, (size_t)L.d * L.f, 1.0f / std::sqrt((float)L.f)));
        L.down.push_back(randn_fp16(rng, (size_t)L.f * L.d, 1.0f / std::sqrt((float)L.d)));
    }
    L.shared_gate = randn_fp16(rng, (size_t)L.d * L.fs, 1.0f / std::sqrt((float)L.fs));
    L.shared_up = randn_fp16(rng, (size_t)L.d * L.fs, 1.0f / std::sqrt((float)L.fs));
    L.shared_down = randn_fp16(rng, (size_t)L.fs * L.d, 1.0f / std::sqrt((float)L.d));
    L.logits.assign((size_t)L.T * L.E, 0);
#pragma omp parallel for
    for (int t = 0; t < L.T; ++t)
        for (int e = 0; e < L.E; ++e) {
            float acc = 0.f;
            for (int j = 0; j < L.d; ++j) acc += h2f(L.x[(size_t)t * L.d + j]) * h2f(router[(size_t)e * L.d + j]);
            L.logits[(size_t)t * L.E + e] = f2h(acc);
        }
    return L;
}

// The stage oracle (tests/moe/moe_topk_test.cpp:198-351 restated): route, stable sort by expert
// (src/moe/moe.cpp:119-126), offsets (src/moe/moe_topk_kernel.cpp:152-172), gather (:174-213), expert FFNs,
// shared expert, combine out[t] = sum_i w[t,i] * Y[rev[i*T+t]] + S[t] (:215-251) accumulated in fp32.
Stages reference_stages(const Layer& L) {
    Stages s;
    const int T = L.T, d = L.d, f = L.f, E = L.E, K = L.K, TK = T * K;
    route(L.logits, T, E, K, s);
    std::vector<int> order(TK);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(),
                     [&](int a, int b) { return s.seq_experts_index[a] < s.seq_experts_index[b]; });
    s.permuted_experts.resize(TK);
    s.permuted_rows.resize(TK);
    s.rev_permuted_rows.resize(TK);
    for (int i = 0; i < TK; ++i) {
        s.permuted_experts[i] = s.seq_experts_index[order[i]];
        s.permuted_rows[i] = s.source_rows[order[i]];
        s.rev_permuted_rows[s.permuted_rows[i]] = i;
    }
    s.first_token_offset.assign(E + 1, 0);
    for (int e = 0; e <= E; ++e)
        s.first_token_offset[e] =
            (int)(std::lower_bound(s.permuted_experts.begin(), s.permuted_experts.end(), e) - s.permuted_experts.begin());
    s.expanded_seq_input.resize((size_t)TK * d);
    s.expanded_seq_softmax.resize(TK);
    for (int i = 0; i < TK; ++i) {
        const int tok = s.permuted_rows[i] % T, rank = s.permuted_rows[i] / T;
        memcpy(&s.expanded_seq_input[(size_t)i * d], &L.x[(size_t)tok * d], (size_t)d * 2);
        s.expanded_seq_softmax[i] = s.seq_experts_softmax[(size_t)tok * K + rank];
    }
    s.expanded_fc1_output.assign((size_t)TK * f, 0);
    s.expanded_fc2_output.assign((size_t)TK * d, 0);
    std::vector<uint16_t> g, u;
    for (int e = 0; e < E; ++e) {
        const int a = s.first_token_offset[e], b = s.first_token_offset[e + 1];
        if (b <= a) continue;
        const size_t rows = (size_t)(b - a);
        g.resize(rows * f);
        u.resize(rows * f);
        linear_fp16(&s.expanded_seq_input[(size_t)a * d], rows, d, L.gate[e].data(), f, g.data());
        linear_fp16(&s.expanded_seq_input[(size_t)a * d], rows, d, L.up[e].data(), f, u.data());
        swiglu_fp16(g.data(), u.data(), rows * f, &s.expanded_fc1_output[(size_t)a * f]);
        linear_fp16(&s.expanded_fc1_output[(size_t)a * f], rows, f, L.down[e].data(), d, &s.expanded_fc2_output[(size_t)a * d]);
    }
    s.shared_fc1_output.resize((size_t)T * L.fs);
    s.shared_fc2_output.resize((size_t)T * d);
    g.resize((size_t)T * L.fs);
    u.resize((size_t)T * L.fs);
    linear_fp16(L.x.data(), T, d, L.shared_gate.data(), L.fs, g.data());
    linear_fp16(L.x.data(), T, d, L.shared_up.data(), L.fs, u.data());
    swiglu_fp16(g.data(), u.data(), (size_t)T * L.fs, s.shared_fc1_output.data());
    linear_fp16(s.shared_fc1_output.data(), T, L.fs, L.shared_down.data(), d, s.shared_fc2_output.data());
    s.final_output.resize((size_t)T * d);
#pragma omp parallel for
    for (int t = 0; t < T; ++t)
        for (int j = 0; j < d; ++j) {
            float acc = 0.f;
            for (int i = 0; i < K; ++i) {
                const int pos = s.rev_permuted_rows[i * T + t];
                acc += h2f(s.expanded_seq_softmax[pos]) * h2f(s.expanded_fc2_output[(size_t)pos * d + j]);
            }
            s.final_output[(size_t)t * d + j] = f2h(acc + h2f(s.shared_fc2_output[(size_t)t * d + j]));
        }
    return s;
}

// --------------------------------------------------------------------------------- device --
#define CK(call)                                                                                   \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) {                                                                   \
            fprintf(stderr, "%s failed: %s\n", #call, cudaGetErrorString(e_));                     \
            exit(100);                                                                             \
        }                                                                                          \
    } while (0)

struct DeviceArena {
    std::vector<void*> ptrs;
    void* alloc(size_t bytes) {
        void* p = nullptr;
        CK(cudaMalloc(&p, std::max<size_t>(bytes, 16)));
        CK(cudaMemset(p, 0xCD, std::max<size_t>(bytes, 16)));     // stale data must not look like a result
        ptrs.push_back(p);
        return p;
    }
    template <class T>
    void* upload(const std::vector<T>& v) {
        void* p = alloc(v.size() * sizeof(T));
        CK(cudaMemcpy(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
        return p;
    }
    ~DeviceArena() {
        for (void* p : ptrs) cudaFree(p);
    }
};

template <class T>
std::vector<T> download(const void* dev, size_t n) {
    std::vector<T> v(n);
    CK(cudaMemcpy(v.data(), dev, n * sizeof(T), cudaMemcpyDeviceToHost));
    return v;
}

// |r - e| <= atol + rtol * |e|, NaN / Inf must agree: the rule of tests/checker/checker.cpp:10-50.
int compare_fp16(const char* name, const std::vector<uint16_t>& got, const std::vector<uint16_t>& exp, float rtol,
                 float atol) {
    size_t bad = 0, first = 0;
    float worst = 0.f;
    for (size_t i = 0; i < exp.size(); ++i) {
        const float r = h2f(got[i]), e = h2f(exp[i]);
        const bool mismatch = (std::isnan(r) != std::isnan(e)) || (std::isinf(r) != std::isinf(e)) ||
                              (!std::isnan(e) && !std::isinf(e) && std::fabs(r - e) > atol + rtol * std::fabs(e));
        if (mismatch && bad++ == 0) first = i;
        if (std::isfinite(r) && std::isfinite(e)) worst = std::max(worst, std::fabs(r - e));
    }
    if (bad)
        printf("  FAIL %-22s %zu of %zu mismatched (first at %zu: got %g, expected %g), max |err| %g\n", name, bad,
               exp.size(), first, h2f(got[first]), h2f(exp[first]), worst);
    else
        printf("  ok   %-22s %zu values, max |err| %g\n", name, exp.size(), worst);
    return bad ? 1 : 0;
}

int compare_int(const char* name, const std::vector<int>& got, const std::vector<int>& exp) {
    size_t bad = 0, first = 0;
    for (size_t i = 0; i < exp.size(); ++i)
        if (got[i] != exp[i] && bad++ == 0) first = i;
    if (bad)
        printf("  FAIL %-22s %zu of %zu differ (first at %zu: got %d, expected %d)\n", name, bad, exp.size(), first,
               got[first], exp[first]);
    else
        printf("  ok   %-22s %zu values, exact\n", name, exp.size());
    return bad ? 1 : 0;
}

// --dump DIR: inputs and CPU stage tensors of one case as raw little-endian files, so that another
// restatement (the numpy oracle of the Python tests) can be compared with this one without a GPU.
template <class T>
bool dump_vec(const std::string& dir, const char* name, const std::vector<T>& v) {
    const std::string path = dir + "/" + name + ".bin";
    FILE* f = fopen(path.c_str(), "wb");
    if (!f) return false;
    const bool ok = fwrite(v.data(), sizeof(T), v.size(), f) == v.size();
    fclose(f);
    return ok;
}

int dump_case(const InputParams& q, const std::string& dir) {
    const Layer L = make_layer(q);
    const Stages s = reference_stages(L);
    bool ok = dump_vec(dir, "x", L.x) && dump_vec(dir, "logits", L.logits) && dump_vec(dir, "shared_gate", L.shared_gate) &&
              dump_vec(dir, "shared_up", L.shared_up) && dump_vec(dir, "shared_down", L.shared_down);
    for (int e = 0; e < L.E && ok; ++e)
        ok = dump_vec(dir, ("gate" + std::to_string(e)).c_str(), L.gate[e]) &&
             dump_vec(dir, ("up" + std::to_string(e)).c_str(), L.up[e]) &&
             dump_vec(dir, ("down" + std::to_string(e)).c_str(), L.down[e]);
    ok = ok && dump_vec(dir, "seq_experts_index", s.seq_experts_index) && dump_vec(dir, "seq_experts_softmax", s.seq_experts_softmax) &&
         dump_vec(dir, "source_rows", s.source_rows) && dump_vec(dir, "permuted_experts", s.permuted_experts) &&
         dump_vec(dir, "permuted_rows", s.permuted_rows) && dump_vec(dir, "first_token_offset", s.first_token_offset) &&
         dump_vec(dir, "rev_permuted_rows", s.rev_permuted_rows) && dump_vec(dir, "expanded_seq_softmax", s.expanded_seq_softmax) &&
         dump_vec(dir, "expanded_fc1_output", s.expanded_fc1_output) && dump_vec(dir, "expanded_fc2_output", s.expanded_fc2_output) &&
         dump_vec(dir, "shared_fc2_output", s.shared_fc2_output) && dump_vec(dir, "final_output", s.final_output);
    if (!ok) fprintf(stderr, "cannot write into %s\n", dir.c_str());
    return ok ? 0 : 100;
}

typedef int (*run_topk_t)(MoEInputRaw*, rf_stream_t, PerfMetrics*);
typedef int (*status_t)(int*);

int run_case(int index, const InputParams& q, run_topk_t run_topk_fn, status_t status_fn) {
    printf("case %d: batch %d x seq %d, d_hidden %d, d_expert %d, experts %d, top-%d, shared %d, seed %d\n", index,
           q.batch_size, q.seq_len, q.d_hidden, q.d_expert, q.n_routed_experts, q.n_experts_per_token,
           q.n_shared_experts, q.seed);
    const Layer L = make_layer(q);
    const Stages ref = reference_stages(L);
    const int T = L.T, d = L.d, f = L.f, E = L.E, K = L.K, TK = T * K;

    DeviceArena mem;
    std::vector<void*> hg(E), hu(E), hd(E);
    for (int e = 0; e < E; ++e) {
        hg[e] = mem.upload(L.gate[e]);
        hu[e] = mem.upload(L.up[e]);
        hd[e] = mem.upload(L.down[e]);
    }
    MoEInputRaw in;
    memset(&in, 0, sizeof in);
    in.params = q;
    in.expert_weight_gate = hg.data();
    in.expert_weight_up = hu.data();
    in.expert_weight_down = hd.data();
    in.input_seq = mem.upload(L.x);
    in.shared_expert_weight_gate = mem.upload(L.shared_gate);
    in.shared_expert_weight_up = mem.upload(L.shared_up);
    in.shared_expert_weight_down = mem.upload(L.shared_down);
    in.expert_scores = mem.upload(L.logits);
    in.seq_experts_index = mem.alloc((size_t)TK * 4);
    in.seq_experts_softmax = mem.alloc((size_t)TK * 2);
    in.source_rows = mem.alloc((size_t)TK * 4);
    in.permuted_experts = mem.alloc((size_t)TK * 4);
    in.permuted_rows = mem.alloc((size_t)TK * 4);
    in.first_token_offset = mem.alloc((size_t)(E + 1) * 4);
    in.expanded_seq_input = mem.alloc((size_t)TK * d * 2);
    in.expanded_seq_softmax = mem.alloc((size_t)TK * 2);
    in.rev_permuted_rows = mem.alloc((size_t)TK * 4);
    in.expanded_fc1_output = mem.alloc((size_t)TK * f * 2);
    in.expanded_fc2_output = mem.alloc((size_t)TK * d * 2);
    in.shared_fc1_output = mem.alloc((size_t)T * L.fs * 2);
    in.shared_fc2_output = mem.alloc((size_t)T * d * 2);
    in.final_output = mem.alloc((size_t)T * d * 2);

    PerfMetrics pm;
    memset(&pm, 0, sizeof pm);
    const int rc = run_topk_fn(&in, nullptr, &pm);
    CK(cudaDeviceSynchronize());
    int detail = 0;
    const int st = status_fn ? status_fn(&detail) : 0;
    if (rc != 0 || st != 0) {
        printf("  FAIL run_topk returned %d, device status %d (detail %d)\n", rc, st, detail);
        return 1;
    }

    const float rtol = 1e-2f, atol = 1e-2f;        // tests/moe/moe_topk_test.cpp:636-639
    int failed = 0;
    failed += compare_int("seq_experts_index", download<int>(in.seq_experts_index, TK), ref.seq_experts_index);
    failed += compare_fp16("seq_experts_softmax", download<uint16_t>(in.seq_experts_softmax, TK), ref.seq_experts_softmax, rtol, atol);
    failed += compare_int("source_rows", download<int>(in.source_rows, TK), ref.source_rows);
    failed += compare_int("permuted_experts", download<int>(in.permuted_experts, TK), ref.permuted_experts);
    failed += compare_int("permuted_rows", download<int>(in.permuted_rows, TK), ref.permuted_rows);
    failed += compare_int("first_token_offset", download<int>(in.first_token_offset, E + 1), ref.first_token_offset);
    failed += compare_fp16("expanded_seq_input", download<uint16_t>(in.expanded_seq_input, (size_t)TK * d), ref.expanded_seq_input, 0.f, 0.f);
    failed += compare_fp16("expanded_seq_softmax", download<uint16_t>(in.expanded_seq_softmax, TK), ref.expanded_seq_softmax, rtol, atol);
    failed += compare_int("rev_permuted_rows", download<int>(in.rev_permuted_rows, TK), ref.rev_permuted_rows);
    failed += compare_fp16("expanded_fc1_output", download<uint16_t>(in.expanded_fc1_output, (size_t)TK * f), ref.expanded_fc1_output, rtol, atol);
    failed += compare_fp16("expanded_fc2_output", download<uint16_t>(in.expanded_fc2_output, (size_t)TK * d), ref.expanded_fc2_output, rtol, atol);
    failed += compare_fp16("shared_fc2_output", download<uint16_t>(in.shared_fc2_output, (size_t)T * d), ref.shared_fc2_output, rtol, atol);
    failed += compare_fp16("final_output", download<uint16_t>(in.final_output, (size_t)T * d), ref.final_output, rtol, atol);

    printf("  stage times (PerfMetrics, %d entries):", pm.count);
    for (int i = 0; i < pm.count && i < 20; ++i) printf(" %s=%.3fms", pm.entries[i].name, pm.entries[i].time);
    printf("\n");
    return failed;
}

}  // namespace

int main(int argc, char** argv) {
    std::string lib = getenv("RF_B200_LIB") ? getenv("RF_B200_LIB") : "radeonflow_kernels_b200/librf_b200.so";
    int only = -1;
    bool list = false, full = false;
    std::string dump_dir;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "--lib" && i + 1 < argc) lib = argv[++i];
        else if (a == "--dump" && i + 1 < argc) dump_dir = argv[++i];
        else if (a == "-c" && i + 1 < argc) only = atoi(argv[++i]);
        else if (a == "-l") list = true;
        else if (a == "--full") full = true;
        else {
            fprintf(stderr, "usage: %s [--lib PATH] [-c CASE] [-l] [--full] [--dump DIR]\n", argv[0]);
            return 100;
        }
    }
    const InputParams* cases = full ? kFullCases : kSmallCases;
    const int n_cases = full ? (int)(sizeof kFullCases / sizeof kFullCases[0]) : (int)(sizeof kSmallCases / sizeof kSmallCases[0]);
    if (list) {
        for (int i = 0; i < n_cases; ++i)
            printf("%d: tokens %d d_hidden %d d_expert %d experts %d top_k %d shared %d seed %d\n", i,
                   cases[i].batch_size * cases[i].seq_len, cases[i].d_hidden, cases[i].d_expert,
                   cases[i].n_routed_experts, cases[i].n_experts_per_token, cases[i].n_shared_experts, cases[i].seed);
        return 0;
    }
    if (!dump_dir.empty()) {
        if (only < 0 || only >= n_cases) {
            fprintf(stderr, "--dump needs -c CASE\n");
            return 100;
        }
        return dump_case(cases[only], dump_dir);
    }
    void* handle = dlopen(lib.c_str(), RTLD_NOW);
    if (!handle) {
        fprintf(stderr, "cannot open %s: %s\n", lib.c_str(), dlerror());
        return 100;
    }
    run_topk_t run_topk_fn = (run_topk_t)dlsym(handle, "run_topk");
    status_t status_fn = (status_t)dlsym(handle, "rf_device_status");
    if (!run_topk_fn) {
        fprintf(stderr, "cannot load symbol run_topk: %s\n", dlerror());
        return 100;
    }
    int failed = 0, ran = 0;
    for (int i = 0; i < n_cases; ++i) {
        if (only >= 0 && i != only) continue;
        failed += run_case(i, cases[i], run_topk_fn, status_fn);
        ++ran;
    }
    printf("%d case(s), %d failing stage tensor(s)\n", ran, failed);
    return failed > 99 ? 99 : failed;
}
