// Host-side comparison metrics (ko_check_*): they compare a result with expected values the caller
// supplies and never evaluate an operator on the CPU.  Stand in for the element loop of the
// reference's GEMM driver (nn_operators/gemm/main.cu:157-176).
#include <cmath>
#include <limits>

#include "ko_internal.h"

namespace {
inline double worse(double worst, double e) {
    if (std::isnan(e)) return std::numeric_limits<double>::infinity();
    return e > worst ? e : worst;
}
int check_args(const void *got, const void *want, int64_t n, const double *out) {
    KO_REQUIRE(n >= 0 && out != nullptr, KO_ERR_INVALID_ARG, "check: bad count or NULL result");
    KO_REQUIRE(n == 0 || (got != nullptr && want != nullptr), KO_ERR_INVALID_ARG, "check: NULL buffer");
    return KO_OK;
}
}  // namespace

extern "C" {

int ko_check_max_abs_f32(const float *got, const float *want, int64_t n, double *out) {
    if (int st = check_args(got, want, n, out)) return st;
    double worst = 0.0;
    for (int64_t i = 0; i < n; ++i) worst = worse(worst, std::fabs(static_cast<double>(got[i]) - want[i]));
    *out = worst;
    return KO_OK;
}

int ko_check_max_rel_f32(const float *got, const float *want, int64_t n, double floor, double *out) {
    if (int st = check_args(got, want, n, out)) return st;
    KO_REQUIRE(floor > 0.0, KO_ERR_INVALID_ARG, "check: floor must be positive");
    double worst = 0.0;
    for (int64_t i = 0; i < n; ++i) {
        const double w = want[i], den = std::fabs(w) > floor ? std::fabs(w) : floor;
        worst = worse(worst, std::fabs(static_cast<double>(got[i]) - w) / den);
    }
    *out = worst;
    return KO_OK;
}

int ko_check_rel_frobenius_f32(const float *got, const float *want, int64_t n, double *out) {
    if (int st = check_args(got, want, n, out)) return st;
    double num = 0.0, den = 0.0;
    for (int64_t i = 0; i < n; ++i) {
        const double d = static_cast<double>(got[i]) - want[i];
        num += d * d;
        den += static_cast<double>(want[i]) * want[i];
    }
    *out = den > 0.0 ? std::sqrt(num / den) : std::sqrt(num);
    return KO_OK;
}

int ko_check_max_rowsum_err_f32(const float *got, int64_t rows, int32_t cols, double *out) {
    KO_REQUIRE(rows >= 0 && cols >= 0 && out != nullptr, KO_ERR_INVALID_ARG, "check: bad shape or NULL result");
    KO_REQUIRE(rows == 0 || cols == 0 || got != nullptr, KO_ERR_INVALID_ARG, "check: NULL buffer");
    double worst = 0.0;
    for (int64_t r = 0; r < rows; ++r) {
        double s = 0.0;
        for (int32_t c = 0; c < cols; ++c) s += got[r * static_cast<int64_t>(cols) + c];
        worst = worse(worst, std::fabs(s - 1.0));
    }
    *out = worst;
    return KO_OK;
}

}  // extern "C"
