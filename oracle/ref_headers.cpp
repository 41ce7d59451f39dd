// Test infrastructure: a C binding of the reference's OWN host+device headers, compiled where they lie in the
// reference checkout (nothing is copied; `make _ref/libref_headers.so REF=<checkout>` reads them through -I<REF>/src).
// The differential tests drive this library and the C restatement (liborc) with the same random inputs, so the
// restatement of these stages is checked against the reference's compiled code rather than against itself.
//
// Bound here:
//   src/collision/analytical_manifold.hpp:934-966        amf::PrimitivePair (every analytic pair kind)
//   src/nk/solve/augmented_row.hpp:231-251               ComputeFloatScalarResponse, EvaluateScalarImpulse (float)
//   src/nk/solve/augmented_row.hpp:319-363               ConeArgument, EvaluateTangentImpulse
//   src/nk/solve/augmented_row.hpp:111-138               MultiplierMomentumRestart, RelaxContactImpulse
//   src/constraint/solref_solimp.hpp:41-78               ComputeCompliantRowTerms (pins the header for later use)
//   src/constraint/coulomb_contact.hpp:27-95             ProjectedContactNormal, ProjectedCoulombStep
#include <cstdint>
#include <cstring>

#include "collision/analytical_manifold.hpp"
#include "collision/shape_kind.hpp"
#include "constraint/coulomb_contact.hpp"
#include "constraint/solref_solimp.hpp"
#include "nk/solve/augmented_row.hpp"

namespace amf = nuka::collision::amf;
namespace aug = nuka::nk::augmented;
using nuka::math::Vec3;

namespace {
amf::PrimParams make_prim(const float* frame, const float* params) {
    amf::PrimParams p;
    p.frame.cx = {frame[0], frame[1], frame[2]};
    p.frame.cy = {frame[3], frame[4], frame[5]};
    p.frame.cz = {frame[6], frame[7], frame[8]};
    p.frame.t = {frame[9], frame[10], frame[11]};
    // the fill of MakePrim, src/phi/backend_cuda/ops/narrowphase_prims.cu:34-45
    p.radius = params[0];
    p.half_height = params[1];
    p.half_extents = {params[0], params[1], params[2]};
    return p;
}
}  // namespace

extern "C" {

// One analytic pair.  frame = world axes cx, cy, cz then origin t (12 floats); params = shape params (4).
// out: per point position(3) normal(3) penetration(1); keys: stable_key per point.  Returns the point count, or -1
// when the pair kind has no analytic handler.
int ref_manifold_frames(uint32_t kind_a, const float* frame_a, const float* params_a, uint32_t kind_b,
                        const float* frame_b, const float* params_b, float query, float* out, uint64_t* keys) {
    const amf::PrimParams a = make_prim(frame_a, params_a), b = make_prim(frame_b, params_b);
    nuka::constraint::ContactManifold m;
    if (!amf::PrimitivePair(kind_a, a, kind_b, b, query, &m)) return -1;
    for (uint32_t i = 0; i < m.point_count; ++i) {
        const auto& p = m.points[i];
        float* o = out + 7 * i;
        o[0] = p.position.x; o[1] = p.position.y; o[2] = p.position.z;
        o[3] = p.normal.x; o[4] = p.normal.y; o[5] = p.normal.z;
        o[6] = p.penetration;
        keys[i] = p.stable_key;
    }
    return static_cast<int>(m.point_count);
}

// Row laws over n records; `in` is n x in_stride floats, `out` n x out_stride floats.
//   which 0  scalar impulse   in: dual rho residual compliance lower upper        out: impulse curvature
//   which 1  cone argument    in: dual rho mu residual                            out: value
//   which 2  tangent impulse  in: dual_y dual_z rho res_y res_z normal mu1 mu2    out: iy iz cyy czz cyz
//   which 3  momentum restart in: point(3) next(3) base(3) scale(3)               out: value (rounded to float)
//   which 4  relaxation       in: dual(3) next(3) last.step(3) last.weight last.point(3)
//                                                                                 out: relaxed(3) weight
//   which 5  compliant terms  in: solref(2) solimp(5) pos_imp pos_aref vel invweight dt   out: k b imp D R aref
//   which 6  coulomb step     in: response(xx yy zz xy xz yz) residual(3) impulse(3) mu1 mu2   out: step(3)
void ref_law_batch(int which, uint32_t n, const float* in, uint32_t in_stride, float* out, uint32_t out_stride) {
    for (uint32_t i = 0; i < n; ++i) {
        const float* x = in + static_cast<size_t>(i) * in_stride;
        float* o = out + static_cast<size_t>(i) * out_stride;
        if (which == 0) {
            const auto t = aug::EvaluateScalarImpulse(x[0], x[1], x[2], x[3], x[4], x[5], aug::ComputeFloatScalarResponse(x[1], x[3]));
            o[0] = t.impulse; o[1] = t.curvature;
        } else if (which == 1) {
            o[0] = aug::ConeArgument(x[0], x[1], x[2], x[3]);
        } else if (which == 2) {
            const auto t = aug::EvaluateTangentImpulse(Vec3{0.0f, x[0], x[1]}, x[2], Vec3{0.0f, x[3], x[4]}, x[5], x[6], x[7]);
            o[0] = t.impulse.y; o[1] = t.impulse.z; o[2] = t.curvature.yy; o[3] = t.curvature.zz; o[4] = t.curvature.yz;
        } else if (which == 3) {
            o[0] = static_cast<float>(aug::MultiplierMomentumRestart(Vec3{x[0], x[1], x[2]}, Vec3{x[3], x[4], x[5]},
                                                                    Vec3{x[6], x[7], x[8]}, Vec3{x[9], x[10], x[11]}));
        } else if (which == 4) {
            aug::ContactRelaxation last{Vec3{x[6], x[7], x[8]}, x[9], Vec3{x[10], x[11], x[12]}};
            const Vec3 r = aug::RelaxContactImpulse(Vec3{x[0], x[1], x[2]}, Vec3{x[3], x[4], x[5]}, &last);
            o[0] = r.x; o[1] = r.y; o[2] = r.z; o[3] = last.weight;
        } else if (which == 5) {
            const auto t = nuka::constraint::ComputeCompliantRowTerms(x, x + 2, x[7], x[8], x[9], x[10], x[11]);
            o[0] = t.k; o[1] = t.b; o[2] = t.imp; o[3] = t.D; o[4] = t.R; o[5] = t.aref;
        } else if (which == 6) {
            const nuka::math::SymmetricMat3 response(x[0], x[1], x[2], x[3], x[4], x[5]);
            const Vec3 s = nuka::constraint::ProjectedCoulombStep(response, Vec3{x[6], x[7], x[8]}, Vec3{x[9], x[10], x[11]}, x[12], x[13]);
            o[0] = s.x; o[1] = s.y; o[2] = s.z;
        }
    }
}

}  // extern "C"
