// Named tuning-parameter store behind OverrideParameters / RetrieveParameters.
//
// The reference keeps per-device tuning parameters in a database that feeds its JIT compiler
// (src/database/database.cpp:57-182) and lets callers replace a family's values at run time
// (src/api_common.cpp:140-221). Kernels here are compiled ahead of time and chosen by a static table, so the
// store only has to behave the same at the API: families and parameter names are those of the reference,
// an override must name every parameter of its family, unknown families are a database error, and a
// retrieve returns what was last stored. One value is honoured: GemmRoutine/XGEMM_MIN_INDIRECT_SIZE = t makes
// calls with m*n*k < t^3 use the small-tile kernel family, which is how the reference's tests force its
// "direct" path (test/routines/level3/xgemm.hpp:62-70).
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "b200blas.h"
#include "params_store.h"

namespace b200 {

namespace {

using Family = std::vector<std::pair<std::string, size_t>>;

// Parameter names per kernel family (reference: src/database/kernels/*/*.hpp, first line of each table).
// The values describe this library's own kernels where a name has a meaning here (tile extents, vector
// widths, thread-block shape) and are 1 or 0 otherwise.
const std::map<std::string, Family>& families() {
  static const std::map<std::string, Family> table = {
      {"Xgemm",
       {{"GEMMK", 0}, {"KREG", 1}, {"KWG", 16}, {"KWI", 1}, {"MDIMA", 16}, {"MDIMC", 16}, {"MWG", 128}, {"NDIMB", 16},
        {"NDIMC", 16}, {"NWG", 128}, {"SA", 1}, {"SB", 1}, {"STRM", 0}, {"STRN", 0}, {"VWM", 4}, {"VWN", 4}}},
      {"XgemmDirect",
       {{"KWID", 1}, {"MDIMAD", 8}, {"MDIMCD", 8}, {"NDIMBD", 8}, {"NDIMCD", 8}, {"PADA", 1}, {"PADB", 1}, {"VWMD", 4},
        {"VWND", 4}, {"WGD", 32}}},
      {"GemmRoutine", {{"XGEMM_MIN_INDIRECT_SIZE", 0}}},
      {"Xconvgemm",
       {{"KWID", 1}, {"MDIMAD", 16}, {"MDIMCD", 16}, {"NDIMBD", 16}, {"NDIMCD", 16}, {"PADA", 1}, {"PADB", 1},
        {"VWMD", 4}, {"VWND", 4}, {"WGD", 128}}},
      {"Copy", {{"COPY_DIMX", 8}, {"COPY_DIMY", 8}, {"COPY_VW", 1}, {"COPY_WPT", 1}}},
      {"Pad", {{"PAD_DIMX", 8}, {"PAD_DIMY", 8}, {"PAD_WPTX", 1}, {"PAD_WPTY", 1}}},
      {"Transpose", {{"TRA_DIM", 8}, {"TRA_PAD", 0}, {"TRA_SHUFFLE", 0}, {"TRA_WPT", 1}}},
      {"Padtranspose", {{"PADTRA_PAD", 0}, {"PADTRA_TILE", 8}, {"PADTRA_WPT", 1}}},
  };
  return table;
}

bool known_precision(int p) { return p == 16 || p == 32 || p == 64 || p == 3232 || p == 6464; }

std::mutex g_mutex;
std::map<std::tuple<int, std::string, int>, Family> g_overrides;

const Family* lookup(int device, const std::string& kernel, int precision) {
  auto it = g_overrides.find(std::make_tuple(device, kernel, precision));
  if (it != g_overrides.end()) return &it->second;
  auto fit = families().find(kernel);
  return fit == families().end() ? nullptr : &fit->second;
}

}  // namespace

size_t min_indirect_size(int device, int precision) {
  std::lock_guard<std::mutex> lock(g_mutex);
  const Family* fam = lookup(device, "GemmRoutine", precision);
  return fam ? (*fam)[0].second : 0;
}

}  // namespace b200

extern "C" int b200blas_override_parameters(int device, const char* kernel_name, int precision,
                                            const char* const* names, const size_t* values, size_t count) {
  using namespace b200;
  if (!kernel_name || (count && (!names || !values))) return -2039;  // kUnexpectedError
  auto fit = families().find(kernel_name);
  if (fit == families().end() || !known_precision(precision)) return -2041;  // kDatabaseError
  Family updated = fit->second;
  for (auto& entry : updated) {
    bool found = false;
    for (size_t i = 0; i < count; ++i) {
      if (entry.first == names[i]) {
        entry.second = values[i];
        found = true;
        break;
      }
    }
    if (!found) return -2047;  // kMissingOverrideParameter
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  g_overrides[std::make_tuple(device, std::string(kernel_name), precision)] = updated;
  return 0;
}

extern "C" int b200blas_retrieve_parameters(int device, const char* kernel_name, int precision, const char** names,
                                            size_t* values, size_t capacity, size_t* count) {
  using namespace b200;
  if (!kernel_name || !count) return -2039;
  if (!known_precision(precision)) return -2041;
  std::lock_guard<std::mutex> lock(g_mutex);
  const Family* fam = lookup(device, kernel_name, precision);
  if (!fam) return -2041;
  *count = fam->size();
  for (size_t i = 0; i < fam->size() && i < capacity; ++i) {
    if (names) names[i] = (*fam)[i].first.c_str();
    if (values) values[i] = (*fam)[i].second;
  }
  return 0;
}
