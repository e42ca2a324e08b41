// Tolerant comparison of two k-NN results, with the semantics of the reference's `--verify`
// (src/verify.cpp:16-112): runs of approximately equal distances are put into one label
// order in both results first; a remaining label mismatch is forgiven only when the rest of
// that query's row is one tie group in both results and the distances at the slot agree.
#include <cmath>
#include <cstdint>
#include <iostream>
#include <limits>

#include "bitsknn/knn.hpp"

namespace bits
{

namespace
{

constexpr float EPSILON = 1e-3F;

bool close(float a, float b)
{
    if (a == b)
    {
        return true;
    }
    const float magnitude = std::fabs(a) + std::fabs(b);
    const float diff = std::fabs(a - b);
    const float tiny = std::numeric_limits<float>::min();
    if (a == 0 || b == 0 || magnitude < tiny)
    {
        return diff < EPSILON * tiny;
    }
    return diff / std::fmin(magnitude, std::numeric_limits<float>::max()) < EPSILON;
}

void order_tie_runs(std::vector<distance_pair>& data)
{
    for (std::int64_t i = 1; i < static_cast<std::int64_t>(data.size()); ++i)
    {
        for (std::int64_t j = i; j > 0 && close(data[j].distance, data[j - 1].distance) &&
                                 data[j].index > data[j - 1].index;
             --j)
        {
            std::swap(data[j], data[j - 1]);
        }
    }
}

bool single_tie_group(const std::vector<distance_pair>& data, std::size_t begin, std::size_t end)
{
    if (begin == end)
    {
        return false;
    }
    for (std::size_t i = begin + 1; i < end; ++i)
    {
        if (!close(data[i - 1].distance, data[i].distance))
        {
            return false;
        }
    }
    return true;
}

} // namespace

bool verify(const std::vector<distance_pair>& expected_result, const std::vector<distance_pair>& actual_result,
            std::size_t k)
{
    auto expected = expected_result;
    auto actual = actual_result;
    order_tie_runs(expected);
    order_tie_runs(actual);
    bool same = expected.size() == actual.size();
    for (std::size_t i = 0; i < expected.size() && i < actual.size(); ++i)
    {
        if (expected[i].index == actual[i].index)
        {
            continue;
        }
        const std::size_t row_end = i + (k - (i % k));
        if (single_tie_group(expected, i, row_end) && single_tie_group(actual, i, row_end) &&
            close(expected[i].distance, actual[i].distance))
        {
            continue;
        }
        std::cerr << "Difference at index " << i << " (expected: " << expected[i].index
                  << ", actual: " << actual[i].index << ")" << '\n';
        std::cerr << "- expected distance: " << expected[i].distance << '\n';
        std::cerr << "- actual distance: " << actual[i].distance << '\n';
        same = false;
    }
    return same;
}

} // namespace bits
