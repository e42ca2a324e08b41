// Host-layer self test: an expired device-side wait must surface as an exception from the
// phase that follows it, not as a silently incomplete result.  Run on a GPU; prints "ok".
#include <cstdio>
#include <cstring>
#include <random>
#include <stdexcept>
#include <vector>

#include "bitsknn/knn.hpp"

int main()
{
    try
    {
        const std::size_t n = 20000, q = 8, dim = 4, k = 16;
        std::mt19937 rng{5};
        std::uniform_real_distribution<float> uni{0.0F, 1.0F};
        std::vector<float> points(n * dim), queries(q * dim);
        for (auto& v : points)
        {
            v = uni(rng);
        }
        for (auto& v : queries)
        {
            v = uni(rng);
        }
        bits::knn_args args{};
        args.points = points.data();
        args.queries = queries.data();
        args.point_count = n;
        args.query_count = q;
        args.dim = dim;
        args.points_layout = bits::matrix_layout::row_major;
        args.queries_layout = bits::matrix_layout::row_major;
        args.dist_layout = bits::matrix_layout::row_major;
        args.dist_block_size = 256;
        args.selection_block_size = 256;
        args.k = k;
        args.items_per_thread = {1, 1, 1};
        args.deg = 1;
        for (const char* id : {"bits", "bits-sq", "fused-cache", "partial-bitonic-regs", "bits-sharded"})
        {
            std::unique_ptr<bits::knn> alg;
            for (auto& candidate : bits::make_registry())
            {
                if (candidate->id() == id)
                {
                    alg = std::move(candidate);
                }
            }
            if (alg == nullptr)
            {
                std::printf("algorithm %s is not registered\n", id);
                return 1;
            }
            alg->initialize(args);
            alg->distances();
            alg->selection();
            const auto good = alg->finish();
            // a kernel that gives up a bounded wait (the library's diagnostic kernel does so on purpose,
            // within a millisecond, and returns normally) ...
            bits::abi_check(bitsknn_selftest_bounded_wait(nullptr));
            bool thrown = false;
            try
            {
                alg->selection(); // ... must make the phase that follows it throw
            }
            catch (const std::runtime_error& err)
            {
                thrown = std::strstr(err.what(), "bounded wait") != nullptr;
            }
            if (!thrown)
            {
                std::printf("%s: selection() after an expired wait did not throw\n", id);
                return 1;
            }
            alg->selection(); // the status is cleared and the context usable: same result again
            const auto again = alg->finish();
            if (again.size() != good.size() ||
                std::memcmp(again.data(), good.data(), good.size() * sizeof(bits::distance_pair)) != 0)
            {
                std::printf("%s: result changed after the reported timeout\n", id);
                return 1;
            }
        }
        std::printf("ok\n");
        return 0;
    }
    catch (const std::exception& err)
    {
        std::printf("unexpected exception: %s\n", err.what());
        return 1;
    }
}
