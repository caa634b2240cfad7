/* TEST INFRASTRUCTURE. Force-included (g++ -include) in front of the reference's
 * unmodified extension/llm/sampler/sampler.cpp to pin the tie order of the sort at
 * sampler.cpp:148: std::sort leaves the order of equal probabilities unspecified,
 * std::stable_sort keeps the index-ascending order of the candidate array built at
 * sampler.cpp:137-143. */
#include <algorithm>
#include <cmath>
#include <memory>
#define sort stable_sort
