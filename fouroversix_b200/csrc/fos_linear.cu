// A linear layer's forward pass on a packed weight as one host call: amax pass, activation quantization, alpha and
// the FP4 GEMM enqueued from C, the packed activation in a caller-provided workspace. What the calls do is in
// fos_quantize / fos_gemm_alpha / fos_gemm_nvfp4; this entry exists because a layer that is launched call by call
// from an interpreter is bound by the interpreter at decode sizes (16 x 8192 -> 8192: 109 us against 23 us of
// device time).
#include "fos_common.cuh"

namespace fos {
namespace {

struct LinearWorkspace {
    int64_t rows_p, k_p, codes, sf, amax, alpha, total;    // byte offsets, multiples of 256
};

LinearWorkspace linear_workspace(int64_t rows, int64_t k) {
    LinearWorkspace w{};
    w.rows_p = round_up64(rows, 128);
    w.k_p = round_up64(k, 64);
    int64_t at = 0;
    auto take = [&](int64_t bytes) { const int64_t here = at; at += round_up64(bytes, 256); return here; };
    w.amax = take(4);
    w.alpha = take(4);
    w.codes = take(w.rows_p * w.k_p / 2);
    w.sf = take(w.rows_p * w.k_p / 16);
    w.total = at;
    return w;
}

}  // namespace
}  // namespace fos

extern "C" int64_t fos_linear_workspace_bytes(int64_t rows, int64_t in_features) {
    if (rows <= 0 || in_features <= 0) return FOS_ERR_INVALID_ARGUMENT;
    return fos::linear_workspace(rows, in_features).total;
}

extern "C" int fos_linear_forward(const void *x, int x_dtype, int64_t rows, int64_t in_features, int64_t ld_x,
                                  int activation_rule, const uint8_t *w_codes, const uint8_t *w_sf, const float *w_amax,
                                  int weight_rule, int64_t out_features, void *out, int out_dtype, int64_t ld_out,
                                  void *workspace, int64_t workspace_bytes, const fos_gemm_opts *opts, int32_t *status,
                                  void *stream) {
    using namespace fos;
    if (!x || !w_codes || !w_sf || !w_amax || !out || !workspace || rows <= 0 || in_features <= 0 || out_features <= 0)
        return FOS_ERR_INVALID_ARGUMENT;
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) return FOS_ERR_MISALIGNED;
    const LinearWorkspace w = linear_workspace(rows, in_features);
    if (workspace_bytes < w.total) return FOS_ERR_INVALID_ARGUMENT;
    uint8_t *base = static_cast<uint8_t *>(workspace);
    float *amax = reinterpret_cast<float *>(base + w.amax), *alpha = reinterpret_cast<float *>(base + w.alpha);
    int st = fos_quantize(x, x_dtype, rows, in_features, ld_x, FOS_NVFP4, activation_rule, 0, 0, FOS_SF_TILED, nullptr,
                          base + w.codes, base + w.sf, amax, 0, stream);
    if (st != FOS_OK) return st;
    st = fos_gemm_alpha(amax, FOS_NVFP4, activation_rule, w_amax, FOS_NVFP4, weight_rule, alpha, stream);
    if (st != FOS_OK) return st;
    return fos_gemm_nvfp4_ex(base + w.codes, base + w.sf, w_codes, w_sf, alpha, out, out_dtype, w.rows_p,
                             round_up64(out_features, 128), w.k_p, rows, out_features, ld_out, opts, status, stream);
}
