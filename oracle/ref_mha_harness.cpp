// TEST INFRASTRUCTURE — never linked into, imported by or executed from the product.
// C shim around the reference's one-token attention (MHA2Kernels::operator(), include/kernels_mha.hpp:89-318: fp32,
// AVX2, softmax without a scale factor, key range cut into sub-states of bN tokens that are combined afterwards),
// compiled from the reference's headers where they lie (see Makefile: target _ref_mha).  Used to pin
// oracle.port.decode_attention and to write the golden vectors of tests/golden/.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <sstream>
#include <vector>
// include order of the reference's own user of this header (torch-ext/mha_opt.cpp): misc.hpp brings FORCE_INLINE and
// rndup, and tensorND.hpp relies on <vector> / <functional> having been included before it
#include "misc.hpp"
#include "kernels_mha.hpp"

extern "C" {

// q [B, 1, H, K], k / v [B, H, N, K], out [B, 1, H, K], all fp32 and compact.  bn > 0 sets the sub-state length
// (the reference reads it from the environment when the object is built: kernels_mha.hpp:76).
int ref_mha_decode(const float* q, const float* k, const float* v, float* out, int B, int H, int N, int K, int bn) {
    if (bn > 0) {
        char buf[32];
        snprintf(buf, sizeof(buf), "%d", bn);
        setenv("bN", buf, 1);
    }
    MHA2Kernels mha;
    tensorND<float> q0((void*)q, {B, 1, H, K});
    tensorND<float> k0((void*)k, {B, H, N, K});
    tensorND<float> v0((void*)v, {B, H, N, K});
    tensorND<float> wv0((void*)out, {B, 1, H, K});
    mha(q0, k0, v0, wv0, /*kv_head_transposed=*/true, /*with_causal_mask=*/false);
    return 0;
}

}  // extern "C"
