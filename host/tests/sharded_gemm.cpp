// Two (or more) processes, one per GPU: each builds a tbn::ShardedGemm, exchanges the result handles through files,
// multiplies, and checks that its own copy of C -- its own slab and the slabs the peers wrote over NVLink -- equals
// the single-GPU product of the whole weight matrix, bit for bit.
//   sharded_gemm <rank> <world> <scratch dir> [M K N]        (run with TBN_DEVICE=<rank>)
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <string>
#include <thread>
#include <vector>

#include "tbn/tbn.hpp"

static bool file_ready(const std::string& path, size_t bytes) {
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    return f && static_cast<size_t>(f.tellg()) >= bytes;
}

// Host barrier through marker files: every rank writes <dir>/<tag>.<rank> and waits (bounded) for all of them.
static bool barrier(const std::string& dir, const std::string& tag, int rank, int world) {
    { std::ofstream f(dir + "/" + tag + "." + std::to_string(rank)); f << "x"; }
    for (int r = 0; r < world; ++r) {
        const std::string path = dir + "/" + tag + "." + std::to_string(r);
        int tries = 0;
        while (!file_ready(path, 1)) {
            if (++tries > 6000) return false;   // 60 s
            std::this_thread::sleep_for(std::chrono::milliseconds(10));
        }
    }
    return true;
}

int main(int argc, char** argv) {
    using namespace tbn;
    try {
        if (argc < 4) { std::fprintf(stderr, "usage: sharded_gemm rank world dir [M K N]\n"); return 2; }
        const int rank = std::atoi(argv[1]), world = std::atoi(argv[2]);
        const std::string dir = argv[3];
        const int64_t M = argc > 6 ? std::atoll(argv[4]) : 300, K = argc > 6 ? std::atoll(argv[5]) : 640, N = argc > 6 ? std::atoll(argv[6]) : 512;
        // The same A and W on every rank (a small generator, not the point of the test).
        std::uint64_t s = 88172645463325252ull;
        auto rnd = [&]() { s ^= s << 13; s ^= s >> 7; s ^= s << 17; return static_cast<float>(static_cast<int>(s % 20001) - 10000) / 5000.0f; };
        std::vector<float> a(static_cast<size_t>(M) * K), w(static_cast<size_t>(K) * N);
        for (auto& v : a) v = rnd();
        for (auto& v : w) v = rnd();
        Tensor A = make_tensor(Shape{M, K}, a), W = make_tensor(Shape{K, N}, w);
        ShardedGemm sg(rank, world, M, K, N);
        const auto cols = sg.columns();
        const int64_t nc = cols.second - cols.first;
        std::vector<float> slab(static_cast<size_t>(K) * nc);
        for (int64_t k = 0; k < K; ++k) std::memcpy(&slab[k * nc], &w[k * N + cols.first], static_cast<size_t>(nc) * 4);
        sg.set_weights(make_tensor(Shape{K, nc}, slab));
        const ShardedGemm::Handle mine = sg.export_result();
        {
            std::ofstream f(dir + "/handle." + std::to_string(rank) + ".tmp", std::ios::binary);
            f.write(reinterpret_cast<const char*>(mine.data()), 64);
        }
        std::rename((dir + "/handle." + std::to_string(rank) + ".tmp").c_str(), (dir + "/handle." + std::to_string(rank)).c_str());
        if (!barrier(dir, "exported", rank, world)) { std::fprintf(stderr, "rank %d: peers never exported\n", rank); return 3; }
        std::vector<ShardedGemm::Handle> handles(static_cast<size_t>(world));
        for (int r = 0; r < world; ++r) {
            std::ifstream f(dir + "/handle." + std::to_string(r), std::ios::binary);
            f.read(reinterpret_cast<char*>(handles[static_cast<size_t>(r)].data()), 64);
        }
        sg.connect(handles);
        if (!barrier(dir, "connected", rank, world)) return 3;
        sg.multiply(A);               // returns after this rank's kernel has finished (its peer stores included)
        if (!barrier(dir, "multiplied", rank, world)) return 3;
        // Reference on this GPU alone: the whole weight matrix in one call.
        Tensor expect = matmul_float_packed(A, pack_binary_weights(W, 0.0f, false));
        const float* got = sg.result().typed_data<float>();
        const float* want = expect.typed_data<float>();
        size_t bad = 0;
        for (size_t i = 0; i < static_cast<size_t>(M) * N; ++i) bad += std::memcmp(&got[i], &want[i], 4) != 0;
        if (!barrier(dir, "checked", rank, world)) return 3;   // nobody frees its matrix while a peer may still hold it open
        std::printf(bad ? "rank %d: %zu elements differ\n" : "rank %d: sharded gemm ok\n", rank, bad);
        return bad ? 1 : 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "error: %s\n", e.what());
        return 1;
    }
}
