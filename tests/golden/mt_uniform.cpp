// Input generator for the golden fixtures: the reference's tests draw their activations from
// std::mt19937(seed) through std::uniform_real_distribution<float> (tests/test_ops_oracle.cpp:298-302,
// :911-917).  The distribution's mapping is implementation-defined, so the libstdc++ stream produced
// here is written to disk once and the committed arrays are the golden inputs.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

int main(int argc, char** argv) {
    if (argc != 6) { std::fprintf(stderr, "usage: mt_uniform seed lo hi count out.bin\n"); return 2; }
    unsigned seed = static_cast<unsigned>(std::strtoul(argv[1], nullptr, 10));
    float lo = std::strtof(argv[2], nullptr), hi = std::strtof(argv[3], nullptr);
    size_t n = std::strtoull(argv[4], nullptr, 10);
    std::mt19937 rng(seed);
    std::uniform_real_distribution<float> dist(lo, hi);
    std::vector<float> v(n);
    for (auto& x : v) x = dist(rng);
    FILE* f = std::fopen(argv[5], "wb");
    if (!f) return 1;
    std::fwrite(v.data(), sizeof(float), n, f);
    std::fclose(f);
    return 0;
}
