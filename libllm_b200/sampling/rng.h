// Counter-based random numbers.
//
// uniform(seed, sequence, step) is a pure function: the draw for the n-th token of a request does
// not depend on which other requests share its batch or on the slot it got.  The reference seeds
// one generator per process from the clock (src/lutil/random.cc:28-31) or leaves cuRAND's default
// seed (src/flint/cuda/cuda_operators.cc:274-276), so its draws cannot be replayed.
#pragma once
#include <cstdint>
#include <string>

namespace llm {

// The finalizer of SplitMix64.
inline uint64_t splitmix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// A number in [0, 1) with 24 random bits, exactly representable in 32-bit floating point.
inline float uniform(uint64_t seed, uint64_t sequence, uint64_t step) {
  uint64_t h = splitmix64(seed);
  h = splitmix64(h ^ sequence);
  h = splitmix64(h ^ step);
  return (float)(h >> 40) / 16777216.0f;
}

// A seed for one named tensor of a random model: depends on the model's seed and the name alone,
// so a tensor's values do not change with the order of the list or with what else the model has.
inline uint64_t tensor_seed(uint64_t seed, const std::string &name) {
  uint64_t h = 0xcbf29ce484222325ull;          // FNV-1a over the name
  for (unsigned char c : name) h = (h ^ c) * 0x100000001b3ull;
  return splitmix64(splitmix64(seed) ^ h);
}

}  // namespace llm
