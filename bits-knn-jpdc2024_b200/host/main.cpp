// `knn` -- command-line benchmark driver with the reference's surface (src/main.cpp:106-448,
// docs/knn.md): same options and defaults, same CSV rows on stdout
//   algorithm,generator,preprocessor,iteration,point_count,query_count,dim,block_size,k,
//   items_per_thread,deg,phase,time
// (phases prepare, transfer-in, distances, selection, postprocessing, finish, transfer-out),
// the `Checksum:` line on stderr per iteration (sum of query 0's k indices, uint32) and
// `--verify ALG`.  cxxopts is not used; the small parser below accepts the same spellings
// (-a X, -aX, --algorithm X, --algorithm=X, and bare flags).
#include <array>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdlib>
#include <iomanip>
#include <iostream>
#include <limits>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "bitsknn/generators.hpp"
#include <cuda_runtime_api.h>

#include "bitsknn/knn.hpp"

namespace
{

struct option_spec
{
    char short_name; // 0 = none
    const char* long_name;
    const char* help;
    const char* default_value; // nullptr = flag without a value
};

const option_spec OPTIONS[] = {
    {'a', "algorithm", "Used algorithm", "serial"},
    {'r', "repeat", "Number of executions", "1"},
    {'k', "knn", "Number of nearest neighbors", "1"},
    {'n', "number", "Number of objects in the database", "1024"},
    {'q', "query", "Number of query objects", "1024"},
    {'d', "dimension", "Dimension of objects", "1"},
    {'g', "generator", "Data generator", "uniform"},
    {'p', "preprocessor", "Data preprocessor", "identity"},
    {0, "seed", "Seed for the data generator", "0"},
    {0, "block-size", "Block size for CUDA kernels", "256"},
    {0, "items-per-thread", "Number of items per thread in the fused-regs kernel (two comma separated values)", "1"},
    {'v', "verify", "Verify the results against selected implementation", "off"},
    {0, "point-layout", "Layout of the point matrix - \"column\" for column major or \"row\" for row major", "row"},
    {0, "query-layout", "Layout of the query matrix - \"column\" for column major or \"row\" for row major", "row"},
    {0, "deg", "degree of parallelism used for single-query problems", "1"},
    {0, "no-output", "Do not copy the result back to CPU", nullptr},
    {0, "header", "Print header with column names and exit", nullptr},
    {'h', "help", "Show help message and exit", nullptr},
};

struct parsed_options
{
    std::map<std::string, std::string> values;
    std::map<std::string, int> counts;

    const std::string& operator[](const std::string& name) const { return values.at(name); }
    int count(const std::string& name) const
    {
        const auto it = counts.find(name);
        return it == counts.end() ? 0 : it->second;
    }
};

const option_spec* find_long(const std::string& name)
{
    for (const auto& opt : OPTIONS)
    {
        if (name == opt.long_name)
        {
            return &opt;
        }
    }
    return nullptr;
}

const option_spec* find_short(char name)
{
    for (const auto& opt : OPTIONS)
    {
        if (opt.short_name != 0 && opt.short_name == name)
        {
            return &opt;
        }
    }
    return nullptr;
}

parsed_options parse(int argc, char** argv)
{
    parsed_options result;
    for (const auto& opt : OPTIONS)
    {
        result.values[opt.long_name] = opt.default_value != nullptr ? opt.default_value : "false";
    }
    for (int i = 1; i < argc; ++i)
    {
        const std::string arg = argv[i];
        const option_spec* opt = nullptr;
        std::string value;
        bool has_value = false;
        if (arg.rfind("--", 0) == 0)
        {
            const auto eq = arg.find('=');
            opt = find_long(arg.substr(2, eq == std::string::npos ? std::string::npos : eq - 2));
            if (eq != std::string::npos)
            {
                value = arg.substr(eq + 1);
                has_value = true;
            }
        }
        else if (arg.size() >= 2 && arg[0] == '-')
        {
            opt = find_short(arg[1]);
            if (arg.size() > 2)
            {
                value = arg.substr(2);
                has_value = true;
            }
        }
        if (opt == nullptr)
        {
            throw std::invalid_argument("Option '" + arg + "' does not exist");
        }
        if (opt->default_value == nullptr)
        {
            result.values[opt->long_name] = "true";
        }
        else
        {
            if (!has_value)
            {
                if (i + 1 >= argc)
                {
                    throw std::invalid_argument(std::string("Option '") + opt->long_name + "' is missing an argument");
                }
                value = argv[++i];
            }
            result.values[opt->long_name] = value;
        }
        ++result.counts[opt->long_name];
    }
    return result;
}

// "1k" = 2^10, "1M" = 2^20, "1G" = 2^30 (reference: include/bits/utils.hpp:20-46)
std::size_t parse_number(std::string number)
{
    if (number.empty())
    {
        return 0;
    }
    std::size_t multiplier = 1;
    switch (number.back())
    {
    case 'k':
    case 'K':
        multiplier = std::size_t{1} << 10U;
        number.pop_back();
        break;
    case 'm':
    case 'M':
        multiplier = std::size_t{1} << 20U;
        number.pop_back();
        break;
    case 'g':
    case 'G':
        multiplier = std::size_t{1} << 30U;
        number.pop_back();
        break;
    default:
        break;
    }
    return static_cast<std::size_t>(std::atol(number.c_str())) * multiplier;
}

// up to three comma separated numbers, missing ones are 1 (utils.hpp:48-74)
std::array<std::size_t, 3> parse_dim3(const std::string& text)
{
    std::array<std::size_t, 3> result{1, 1, 1};
    std::size_t begin = 0;
    for (std::size_t part = 0; part < 3 && begin <= text.size(); ++part)
    {
        const std::size_t end = std::min(text.find(',', begin), text.size());
        result[part] = parse_number(text.substr(begin, end - begin));
        begin = end + 1;
    }
    return result;
}

void print_help(const std::vector<std::unique_ptr<bits::knn>>& algorithms)
{
    std::cerr << "kNN\nUsage:\n  knn [OPTION...]\n\n";
    for (const auto& opt : OPTIONS)
    {
        std::string names = opt.short_name != 0 ? std::string("  -") + opt.short_name + ", --" : std::string("      --");
        names += opt.long_name;
        if (opt.default_value != nullptr)
        {
            names += " arg";
        }
        std::cerr << std::left << std::setw(28) << names << opt.help;
        if (opt.default_value != nullptr)
        {
            std::cerr << " (default: " << opt.default_value << ")";
        }
        std::cerr << '\n';
    }
    std::cerr << '\n' << "Available algorithms:" << '\n';
    for (const auto& alg : algorithms)
    {
        std::cerr << "- " << alg->id() << "\n";
    }
}

void print_log_header()
{
    std::cout << "algorithm,generator,preprocessor,iteration,point_count,query_count,dim,"
                 "block_size,k,items_per_thread,deg,phase,time"
              << '\n';
}

void log(const bits::knn_args& args, const std::string& algorithm, const std::string& generator,
         const std::string& preprocessor, const std::string& phase, std::size_t iteration, double time)
{
    const auto default_precision = std::cout.precision();
    std::cout << algorithm << "," << generator << "," << preprocessor << "," << iteration << "," << args.point_count
              << "," << args.query_count << "," << args.dim << "," << args.selection_block_size << "," << args.k
              << ",\"" << args.items_per_thread[0] << "," << args.items_per_thread[1] << ","
              << args.items_per_thread[2] << "\"," << args.deg << "," << phase << "," << std::scientific
              << std::setprecision(std::numeric_limits<double>::digits10 + 1) << time << std::defaultfloat
              << std::setprecision(static_cast<int>(default_precision)) << '\n';
}

std::vector<float> transpose(const float* matrix, std::size_t row_count, std::size_t col_count)
{
    std::vector<float> result(row_count * col_count);
    for (std::size_t i = 0; i < row_count; ++i)
    {
        for (std::size_t j = 0; j < col_count; ++j)
        {
            result[j * row_count + i] = matrix[i * col_count + j];
        }
    }
    return result;
}

template <class Clock = std::chrono::steady_clock, class Fn>
double timed(Fn&& fn)
{
    const auto start = Clock::now();
    fn();
    const std::chrono::duration<double> elapsed = Clock::now() - start;
    return elapsed.count();
}

} // namespace

int main(int argc, char** argv)
try
{
    auto algorithms = bits::make_registry();

    std::vector<std::unique_ptr<bits::data_generator>> generators;
    generators.push_back(std::make_unique<bits::uniform_generator>());
    generators.push_back(std::make_unique<bits::normal_generator>());
    generators.push_back(std::make_unique<bits::clustered_generator>());

    std::vector<std::unique_ptr<bits::data_preprocessor>> preprocessors;
    preprocessors.push_back(std::make_unique<bits::identity_preprocessor>());
    preprocessors.push_back(std::make_unique<bits::ordering_preprocessor<std::less<>>>("ascending"));
    preprocessors.push_back(std::make_unique<bits::ordering_preprocessor<std::greater<>>>("descending"));

    const auto params = parse(argc, argv);

    if (params.count("help") != 0)
    {
        print_help(algorithms);
        return 0;
    }
    if (params.count("header") != 0)
    {
        print_log_header();
        return 0;
    }

    const std::size_t dim = parse_number(params["dimension"]);
    const std::size_t k = parse_number(params["knn"]);
    const std::size_t input_size = parse_number(params["number"]);
    const std::size_t query_size = parse_number(params["query"]);
    const std::size_t repeat_count = parse_number(params["repeat"]);
    const std::size_t seed = parse_number(params["seed"]);
    const std::string algorithm_id = params["algorithm"];
    std::string generator_id = params["generator"];
    const std::string preprocessor_id = params["preprocessor"];
    const std::size_t block_size = parse_number(params["block-size"]);
    const std::string verify_alg = params["verify"];
    const std::string layout_points = params["point-layout"];
    const std::string layout_queries = params["query-layout"];
    const auto items_per_thread = parse_dim3(params["items-per-thread"]);

    if (dim <= 0)
    {
        std::cerr << "Dimension must be greater than 0" << '\n';
        return 1;
    }
    if (input_size <= 0)
    {
        std::cerr << "Number of objects in the database must be greater than 0" << '\n';
        return 1;
    }
    if (query_size <= 0)
    {
        std::cerr << "Number of query objects must be greater than 0" << '\n';
        return 1;
    }
    if (k <= 0)
    {
        std::cerr << "Number of nearest neighbors must be greater than 0" << '\n';
        return 1;
    }
    if (block_size <= 0)
    {
        std::cerr << "Block size must be greater than 0" << '\n';
        return 1;
    }

    std::string generator_params;
    const auto generator_sep = generator_id.find(':');
    if (generator_sep != std::string::npos)
    {
        generator_params = generator_id.substr(generator_sep + 1);
        generator_id = generator_id.substr(0, generator_sep);
    }
    bits::data_generator* generator = nullptr;
    for (auto& gen : generators)
    {
        if (gen->id() == generator_id)
        {
            generator = gen.get();
        }
    }
    if (generator == nullptr)
    {
        std::cerr << "Unknown generator: '" << generator_id << "'" << '\n';
        return 1;
    }
    generator->set_seed(seed);
    if (generator_sep != std::string::npos)
    {
        generator->set_params(generator_params);
    }
    auto data = generator->generate(input_size, dim);
    auto query = generator->generate(query_size, dim);

    bits::data_preprocessor* preprocessor = nullptr;
    for (auto& pre : preprocessors)
    {
        if (pre->id() == preprocessor_id)
        {
            preprocessor = pre.get();
        }
    }
    if (preprocessor == nullptr)
    {
        std::cerr << "Unknown preprocessor: '" << preprocessor_id << "'" << '\n';
        return 1;
    }
    preprocessor->preprocess(data, query, dim);

    bits::knn_args args{};
    args.points = data.data();
    args.queries = query.data();
    args.point_count = input_size;
    args.query_count = query_size;
    args.dim = dim;
    args.points_layout = layout_points == "row" ? bits::matrix_layout::row_major : bits::matrix_layout::column_major;
    args.queries_layout = layout_queries == "row" ? bits::matrix_layout::row_major : bits::matrix_layout::column_major;
    args.dist_layout = bits::matrix_layout::row_major;
    args.dist_block_size = block_size;
    args.selection_block_size = block_size;
    args.k = k;
    args.items_per_thread = items_per_thread;
    args.deg = parse_number(params["deg"]);

    if (args.points_layout == bits::matrix_layout::column_major)
    {
        data = transpose(data.data(), args.point_count, args.dim);
        args.points = data.data();
    }
    if (args.queries_layout == bits::matrix_layout::column_major)
    {
        query = transpose(query.data(), args.query_count, args.dim);
        args.queries = query.data();
    }

    const bool no_output = params["no-output"] == "true";

    bits::knn* alg = nullptr;
    for (auto& candidate : algorithms)
    {
        if (candidate->id() == algorithm_id)
        {
            alg = candidate.get();
        }
    }
    if (alg == nullptr)
    {
        std::cerr << "Unknown algorithm: '" << algorithm_id << "'" << '\n';
        print_help(algorithms);
        return 1;
    }
    if (no_output)
    {
        alg->no_output();
    }
    // Page-lock the generated inputs (best effort): the uploads of initialize() then run at the
    // bus rate and asynchronously, so the first distance computation overlaps them piece by piece.
    // The reference uploads from pageable vectors (src/distance/magma_distance.cu:52-70).
    const bool locked_points =
        cudaHostRegister(const_cast<float*>(args.points), args.point_count * args.dim * sizeof(float),
                         cudaHostRegisterDefault) == cudaSuccess;
    const bool locked_queries =
        cudaHostRegister(const_cast<float*>(args.queries), args.query_count * args.dim * sizeof(float),
                         cudaHostRegisterDefault) == cudaSuccess;
    cudaGetLastError(); // a refused registration is not an error of the run
    alg->initialize(args);

    for (std::size_t i = 0; i < repeat_count; ++i)
    {
        std::atomic<std::uint32_t> sink{0};

        log(args, algorithm_id, generator_id, preprocessor_id, "prepare", i, timed([&] { alg->prepare(); }));
        log(args, algorithm_id, generator_id, preprocessor_id, "transfer-in", i, alg->transfer_in_seconds());
        log(args, algorithm_id, generator_id, preprocessor_id, "distances", i, timed([&] { alg->distances(); }));
        log(args, algorithm_id, generator_id, preprocessor_id, "selection", i, timed([&] { alg->selection(); }));
        log(args, algorithm_id, generator_id, preprocessor_id, "postprocessing", i,
            timed([&] { alg->postprocessing(); }));
        std::vector<bits::distance_pair> result;
        log(args, algorithm_id, generator_id, preprocessor_id, "finish", i, timed([&] { result = alg->finish(); }));
        log(args, algorithm_id, generator_id, preprocessor_id, "transfer-out", i, alg->transfer_out_seconds());

        if (!no_output)
        {
            for (std::size_t j = 0; j < k && j < result.size(); ++j)
            {
                sink += static_cast<std::uint32_t>(result[j].index);
            }
            std::cerr << "Checksum: " << sink << '\n';
        }

        if (params.count("verify") != 0)
        {
            for (auto& other_alg : algorithms)
            {
                if (other_alg->id() != verify_alg)
                {
                    continue;
                }
                other_alg->initialize(args);
                other_alg->prepare();
                other_alg->distances();
                other_alg->selection();
                const auto expected_result = other_alg->finish();
                bits::verify(expected_result, result, k);
            }
        }
    }
    cudaDeviceSynchronize();
    if (locked_points)
    {
        cudaHostUnregister(const_cast<float*>(args.points));
    }
    if (locked_queries)
    {
        cudaHostUnregister(const_cast<float*>(args.queries));
    }
    return 0;
}
catch (std::exception& e)
{
    std::cerr << e.what() << '\n';
    return 1;
}
catch (...)
{
    std::cerr << "Unknown exception" << '\n';
    return 1;
}
