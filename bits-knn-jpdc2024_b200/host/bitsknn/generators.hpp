// Data generators and preprocessors of the `knn` command line.
//
// `uniform[:min,max]` and `normal[:mean,std]` follow the reference's protocol exactly -- one
// std::default_random_engine seeded once, discard(4096), points drawn before queries, a fresh
// distribution object per matrix (include/bits/generator/uniform_generator.hpp:42-59,
// normal_generator.hpp:42-59, src/main.cpp:291-298) -- so that published checksums reproduce
// with libstdc++.  `clustered:centers,sigma` is an addition: points and queries around
// `centers` uniform centres with Gaussian noise.  Preprocessors: identity, ascending,
// descending (include/bits/preprocessor/ordering_preprocessor.hpp:36-42).
#ifndef BITSKNN_HOST_GENERATORS_HPP_
#define BITSKNN_HOST_GENERATORS_HPP_

#include <algorithm>
#include <cstddef>
#include <cstdlib>
#include <functional>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

namespace bits
{

inline std::vector<float> parse_floats(const std::string& text)
{
    std::vector<float> values;
    std::size_t begin = 0;
    while (begin <= text.size())
    {
        const std::size_t end = std::min(text.find(',', begin), text.size());
        if (end > begin)
        {
            values.push_back(std::strtof(text.substr(begin, end - begin).c_str(), nullptr));
        }
        begin = end + 1;
    }
    return values;
}

class data_generator
{
public:
    virtual ~data_generator() = default;
    virtual std::string id() const = 0;
    virtual std::vector<float> generate(std::size_t count, std::size_t dim) = 0;
    virtual void set_params(const std::string& params) = 0;

    // seed 0 = non-deterministic, as in the reference
    void set_seed(std::size_t seed)
    {
        std::random_device dev;
        engine_ = std::default_random_engine{
            static_cast<std::default_random_engine::result_type>(seed == 0 ? dev() : seed)};
        engine_.discard(1U << 12U);
    }

protected:
    std::default_random_engine engine_;
};

class uniform_generator : public data_generator
{
public:
    std::string id() const override { return "uniform"; }
    std::vector<float> generate(std::size_t count, std::size_t dim) override
    {
        std::uniform_real_distribution<float> dist{min_, max_};
        std::vector<float> data(count * dim);
        for (auto& value : data)
        {
            value = dist(engine_);
        }
        return data;
    }
    void set_params(const std::string& params) override
    {
        const auto values = parse_floats(params);
        if (values.size() > 2)
        {
            throw std::invalid_argument("Invalid number of parameters");
        }
        const float lo = values.size() == 2 ? values[0] : 0.0F;
        const float hi = values.size() == 2 ? values[1] : (values.size() == 1 ? values[0] : max_);
        if (!values.empty())
        {
            if (lo >= hi)
            {
                throw std::invalid_argument("Invalid parameter values");
            }
            min_ = lo;
            max_ = hi;
        }
    }

private:
    float min_ = 0.0F;
    float max_ = 1.0F;
};

class normal_generator : public data_generator
{
public:
    std::string id() const override { return "normal"; }
    std::vector<float> generate(std::size_t count, std::size_t dim) override
    {
        std::normal_distribution<float> dist{mean_, std_dev_};
        std::vector<float> data(count * dim);
        for (auto& value : data)
        {
            value = dist(engine_);
        }
        return data;
    }
    void set_params(const std::string& params) override
    {
        const auto values = parse_floats(params);
        if (values.size() > 2)
        {
            throw std::invalid_argument("Invalid number of parameters");
        }
        if (values.size() == 2)
        {
            mean_ = values[0];
            std_dev_ = values[1];
        }
        else if (values.size() == 1)
        {
            std_dev_ = values[0];
        }
        if (std_dev_ <= 0)
        {
            throw std::invalid_argument("Invalid standard deviation");
        }
    }

private:
    float mean_ = 0.0F;
    float std_dev_ = 1.0F;
};

// centres are drawn once (on the first generate call), so points and queries share them
class clustered_generator : public data_generator
{
public:
    std::string id() const override { return "clustered"; }
    std::vector<float> generate(std::size_t count, std::size_t dim) override
    {
        if (centres_.size() != centre_count_ * dim)
        {
            std::uniform_real_distribution<float> uni{0.0F, 1.0F};
            centres_.resize(centre_count_ * dim);
            for (auto& value : centres_)
            {
                value = uni(engine_);
            }
        }
        std::uniform_int_distribution<std::size_t> pick{0, centre_count_ - 1};
        std::normal_distribution<float> noise{0.0F, sigma_};
        std::vector<float> data(count * dim);
        for (std::size_t i = 0; i < count; ++i)
        {
            const std::size_t c = pick(engine_);
            for (std::size_t d = 0; d < dim; ++d)
            {
                data[i * dim + d] = centres_[c * dim + d] + noise(engine_);
            }
        }
        return data;
    }
    void set_params(const std::string& params) override
    {
        const auto values = parse_floats(params);
        if (values.size() > 2)
        {
            throw std::invalid_argument("Invalid number of parameters");
        }
        if (!values.empty())
        {
            centre_count_ = static_cast<std::size_t>(values[0]);
        }
        if (values.size() == 2)
        {
            sigma_ = values[1];
        }
        if (centre_count_ == 0 || sigma_ <= 0)
        {
            throw std::invalid_argument("Invalid parameter values");
        }
    }

private:
    std::size_t centre_count_ = 256;
    float sigma_ = 0.05F;
    std::vector<float> centres_;
};

class data_preprocessor
{
public:
    virtual ~data_preprocessor() = default;
    virtual std::string id() const = 0;
    virtual void preprocess(std::vector<float>& data, std::vector<float>& query, std::size_t dim) = 0;
};

class identity_preprocessor : public data_preprocessor
{
public:
    std::string id() const override { return "identity"; }
    void preprocess(std::vector<float>&, std::vector<float>&, std::size_t) override {}
};

// sorts the flat coordinate array and zeroes the queries: with dim 1 every distance row is
// then monotone (descending = every element is a new minimum, the adversarial input)
template <class Ordering>
class ordering_preprocessor : public data_preprocessor
{
public:
    explicit ordering_preprocessor(std::string id) : id_(std::move(id)) {}
    std::string id() const override { return id_; }
    void preprocess(std::vector<float>& data, std::vector<float>& query, std::size_t) override
    {
        std::fill(query.begin(), query.end(), 0.0F);
        std::sort(data.begin(), data.end(), Ordering{});
    }

private:
    std::string id_;
};

} // namespace bits

#endif // BITSKNN_HOST_GENERATORS_HPP_
