// Stand-in used ONLY when the reference's own sources are compiled as a checker (oracle/_ref).
// The reference's parallel_knn.cpp includes this header for its default distance object, an
// Eigen CPU GEMM; Eigen is not available here and the checker always installs its own distance
// object (set_dist_impl) before initialize(), so the default is never constructed at run time.
#ifndef BITS_DISTANCE_EIGEN_DISTANCE_HPP_
#define BITS_DISTANCE_EIGEN_DISTANCE_HPP_

#include <stdexcept>
#include <string>

#include "bits/distance/cuda_distance.hpp"

class eigen_distance : public cuda_distance
{
public:
    std::string name() const override { return "eigen-dist"; }
    void prepare(const knn_args&) override { throw std::runtime_error("eigen-dist is not part of this build"); }
    void compute() override {}
};

#endif
