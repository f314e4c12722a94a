// Driver around the UNMODIFIED reference sources (compiled where they lie, never copied):
// builds a CPU tensor, fills it with Tensor::random(min,max,seed) (Tensor/Tensor.cpp:268-298)
// and writes the raw fp32 elements to stdout. Used only to check the oracle's restatement
// of the reference input generator and to make the committed golden vectors.
// Test infrastructure; not part of the shipped library.
#include "Tensor/Tensor.h"
#include <cstdio>
#include <cstdlib>
#include <thread>
int main(int argc, char** argv) {
    if (argc < 6) { std::fprintf(stderr, "usage: %s rows cols seed min max\n", argv[0]); return 2; }
    const size_t rows = std::strtoull(argv[1], nullptr, 10), cols = std::strtoull(argv[2], nullptr, 10);
    const long seed = std::atol(argv[3]);
    const double lo = std::atof(argv[4]), hi = std::atof(argv[5]);
    BeanTensor::Tensors::Tensor t({rows, cols}, BeanTensor::Casting::DType::Float32, BeanTensor::Tensors::Device::CPU);
    t.random(lo, hi, seed);
    t.sync(); // the fill runs on pool threads; reading without this races with it
    const auto v = t.contents_to_flat_vector<float>();
    std::fwrite(v.data(), sizeof(float), v.size(), stdout);
    std::fprintf(stderr, "threads=%u\n", std::thread::hardware_concurrency());
    return 0;
}
