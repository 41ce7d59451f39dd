/* Oracle math helpers (test infrastructure). Vector/quaternion ops follow the reference's
 * src/math/cuda_vec_ops.cuh and 6x6 spatial ops follow src/math/cuda_spatial_ops.cuh:
 * dense row-major 6x6 transforms with left-to-right accumulation. */
#ifndef ORC_MATH_H
#define ORC_MATH_H

#include <math.h>
#include <float.h>
#include <string.h>

typedef struct { float x, y, z; } v3;
typedef struct { float w, x, y, z; } quat;

static inline v3 V3(float x, float y, float z) { v3 r = {x, y, z}; return r; }
static inline v3 v3ld(const float *p) { return V3(p[0], p[1], p[2]); }
static inline void v3st(float *p, v3 a) { p[0] = a.x; p[1] = a.y; p[2] = a.z; }
static inline v3 vadd(v3 a, v3 b) { return V3(a.x + b.x, a.y + b.y, a.z + b.z); }
static inline v3 vsub(v3 a, v3 b) { return V3(a.x - b.x, a.y - b.y, a.z - b.z); }
static inline v3 vscale(v3 a, float s) { return V3(a.x * s, a.y * s, a.z * s); }
static inline v3 vneg(v3 a) { return V3(-a.x, -a.y, -a.z); }
static inline float vdot(v3 a, v3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
static inline v3 vcross(v3 a, v3 b) {
    return V3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x);
}
static inline float vlen(v3 a) { return sqrtf(vdot(a, a)); }
static inline float vcomp(v3 a, int k) { return k == 0 ? a.x : (k == 1 ? a.y : a.z); }
static inline float rsq(float x) { return 1.0f / sqrtf(x); }

static inline quat Q4(float w, float x, float y, float z) { quat q = {w, x, y, z}; return q; }
static inline quat qld(const float *p) { return Q4(p[0], p[1], p[2], p[3]); }
static inline void qst(float *p, quat q) { p[0] = q.w; p[1] = q.x; p[2] = q.y; p[3] = q.z; }
/* cuda_vec_ops.cuh QuatMul */
static inline quat qmul(quat a, quat b) {
    return Q4(a.w * b.w - a.x * b.x - a.y * b.y - a.z * b.z,
              a.w * b.x + a.x * b.w + a.y * b.z - a.z * b.y,
              a.w * b.y - a.x * b.z + a.y * b.w + a.z * b.x,
              a.w * b.z + a.x * b.y - a.y * b.x + a.z * b.w);
}
/* cuda_vec_ops.cuh QuatNormalizeRsqrt(q, eps): identity when |q|^2 <= eps */
static inline quat qnorm_le(quat q, float eps) {
    float n = q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z;
    if (n <= eps) return Q4(1, 0, 0, 0);
    float i = rsq(n);
    return Q4(q.w * i, q.x * i, q.y * i, q.z * i);
}
/* cuda_vec_ops.cuh QuatNormalizeForwardRsqrt(q, eps): identity when |q|^2 < eps */
static inline quat qnorm_lt(quat q, float eps) {
    float n = q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z;
    if (n < eps) return Q4(1, 0, 0, 0);
    float i = rsq(n);
    return Q4(q.w * i, q.x * i, q.y * i, q.z * i);
}
/* cuda_vec_ops.cuh RotateByQuatNormalized: normalises when |q|^2 > 1e-12 */
static inline v3 qrot(quat q, v3 v) {
    float n = q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z;
    if (n > 1.0e-12f) { float i = rsq(n); q.w *= i; q.x *= i; q.y *= i; q.z *= i; }
    v3 qv = V3(q.x, q.y, q.z);
    v3 t = vscale(vcross(qv, v), 2.0f);
    return vadd(vadd(v, vscale(t, q.w)), vcross(qv, t));
}
static inline v3 qrot_inv(quat q, v3 v) {
    float n = q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z;
    if (n > 1.0e-12f) { float i = rsq(n); q.w *= i; q.x *= i; q.y *= i; q.z *= i; }
    v3 qv = V3(-q.x, -q.y, -q.z);
    v3 t = vscale(vcross(qv, v), 2.0f);
    return vadd(vadd(v, vscale(t, q.w)), vcross(qv, t));
}
/* prims_types.cuh PrimRotate: no normalisation */
static inline v3 qrot_raw(quat q, v3 v) {
    v3 qv = V3(q.x, q.y, q.z);
    v3 t = vscale(vcross(qv, v), 2.0f);
    return vadd(vadd(v, vscale(t, q.w)), vcross(qv, t));
}

/* pose = pos(3) + quat wxyz(4) */
static inline void pose_compose(const float *parent, const float *local, float *out) {
    /* articulation.cu:1152-1158 ComposeTransform */
    v3 p = vadd(v3ld(parent), qrot(qld(parent + 3), v3ld(local)));
    quat r = qnorm_le(qmul(qld(parent + 3), qld(local + 3)), 1.0e-12f);
    v3st(out, p); qst(out + 3, r);
}
/* analytical_manifold.hpp:165-171 ComposeTransformHD: rotation product is not renormalised */
static inline void pose_compose_hd(const float *parent, const float *local, float *out) {
    v3 p = vadd(v3ld(parent), qrot(qld(parent + 3), v3ld(local)));
    quat r = qmul(qld(parent + 3), qld(local + 3));
    v3st(out, p); qst(out + 3, r);
}

/* ---- 3x3 ---- */
typedef struct { float m[9]; } m3;
static inline m3 m3_ident(void) { m3 r = {{1, 0, 0, 0, 1, 0, 0, 0, 1}}; return r; }
static inline m3 m3_T(m3 a) { m3 r = {{a.m[0], a.m[3], a.m[6], a.m[1], a.m[4], a.m[7], a.m[2], a.m[5], a.m[8]}}; return r; }
static inline m3 m3_mul(m3 a, m3 b) {
    m3 o;
    for (int r = 0; r < 3; ++r) for (int c = 0; c < 3; ++c)
        o.m[r * 3 + c] = a.m[r * 3 + 0] * b.m[c + 0] + a.m[r * 3 + 1] * b.m[c + 3] + a.m[r * 3 + 2] * b.m[c + 6];
    return o;
}
/* articulation.cu:91-124 */
static inline m3 m3_from_quat(quat q) {
    float n = q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z;
    if (n <= 1.0e-12f) return m3_ident();
    float i = rsq(n); q.w *= i; q.x *= i; q.y *= i; q.z *= i;
    float xx = q.x * q.x, yy = q.y * q.y, zz = q.z * q.z, xy = q.x * q.y, xz = q.x * q.z, yz = q.y * q.z;
    float wx = q.w * q.x, wy = q.w * q.y, wz = q.w * q.z;
    m3 o = {{1.0f - 2.0f * (yy + zz), 2.0f * (xy - wz), 2.0f * (xz + wy),
             2.0f * (xy + wz), 1.0f - 2.0f * (xx + zz), 2.0f * (yz - wx),
             2.0f * (xz - wy), 2.0f * (yz + wx), 1.0f - 2.0f * (xx + yy)}};
    return o;
}
/* articulation.cu:126-147 */
static inline m3 m3_axis_angle(v3 a, float angle) {
    float l = vdot(a, a);
    if (l <= 1.0e-12f) return m3_ident();
    a = vscale(a, rsq(l));
    float c = cosf(angle), s = sinf(angle), t = 1.0f - c;
    m3 o = {{t * a.x * a.x + c, t * a.x * a.y - s * a.z, t * a.x * a.z + s * a.y,
             t * a.x * a.y + s * a.z, t * a.y * a.y + c, t * a.y * a.z - s * a.x,
             t * a.x * a.z - s * a.y, t * a.y * a.z + s * a.x, t * a.z * a.z + c}};
    return o;
}

/* ---- 6-vectors and 6x6 (cuda_spatial_ops.cuh) ---- */
static inline void z6(float *v) { for (int i = 0; i < 6; ++i) v[i] = 0.0f; }
static inline float dot6(const float *a, const float *b) { float s = 0.0f; for (int i = 0; i < 6; ++i) s += a[i] * b[i]; return s; }
static inline void mat66_mulv(const float *M, const float *v, float *o) {
    for (int r = 0; r < 6; ++r) { float s = 0.0f; for (int c = 0; c < 6; ++c) s += M[r * 6 + c] * v[c]; o[r] = s; }
}
static inline void xf_motion(const float *X, const float *in, float *o) { mat66_mulv(X, in, o); }
static inline void xf_force_T(const float *X, const float *in, float *o) {
    for (int r = 0; r < 6; ++r) { float s = 0.0f; for (int c = 0; c < 6; ++c) s += X[c * 6 + r] * in[c]; o[r] = s; }
}
static inline void xf_inertia_to_parent(const float *X, const float *I, float *o) {
    float t[36];
    for (int r = 0; r < 6; ++r) for (int c = 0; c < 6; ++c) { float s = 0.0f; for (int k = 0; k < 6; ++k) s += I[r * 6 + k] * X[k * 6 + c]; t[r * 6 + c] = s; }
    for (int r = 0; r < 6; ++r) for (int c = 0; c < 6; ++c) { float s = 0.0f; for (int k = 0; k < 6; ++k) s += X[k * 6 + r] * t[k * 6 + c]; o[r * 6 + c] = s; }
}
static inline void motion_cross(const float *l, const float *r, float *o) {
    v3 lw = v3ld(l), lv = v3ld(l + 3), rw = v3ld(r), rv = v3ld(r + 3);
    v3st(o, vcross(lw, rw)); v3st(o + 3, vadd(vcross(lw, rv), vcross(lv, rw)));
}
static inline void force_cross(const float *m, const float *f, float *o) {
    v3 w = v3ld(m), v = v3ld(m + 3), n = v3ld(f), ff = v3ld(f + 3);
    v3st(o, vadd(vcross(w, n), vcross(v, ff))); v3st(o + 3, vcross(w, ff));
}
/* articulation.cu:149-171 MakeMotionTransform(rotation E, translation r): [[E,0],[-E r^x, E]] */
static inline void make_motion_xf(m3 E, v3 r, float *X) {
    for (int i = 0; i < 36; ++i) X[i] = 0.0f;
    for (int a = 0; a < 3; ++a) for (int b = 0; b < 3; ++b) { X[a * 6 + b] = E.m[a * 3 + b]; X[(a + 3) * 6 + b + 3] = E.m[a * 3 + b]; }
    m3 skew = {{0, -r.z, r.y, r.z, 0, -r.x, -r.y, r.x, 0}};
    m3 ll = m3_mul(E, skew);
    for (int a = 0; a < 3; ++a) for (int b = 0; b < 3; ++b) X[(a + 3) * 6 + b] = -ll.m[a * 3 + b];
}

/* symmetric 3x3 stored xx yy zz xy xz yz */
static inline v3 sym_mulv(const float *s, v3 v) {
    return V3(s[0] * v.x + s[3] * v.y + s[4] * v.z, s[3] * v.x + s[1] * v.y + s[5] * v.z, s[4] * v.x + s[5] * v.y + s[2] * v.z);
}

/* compensated float sum, reference block_descent_tile.cuh:15-46 */
typedef struct { float value, error; } tsum;
static inline void tsum_add(tsum *s, float x) {
    volatile float sum = s->value + x;
    volatile float part = sum - s->value;
    s->error += (s->value - (sum - part)) + (x - part);
    s->value = sum;
}
static inline void tsum_addp(tsum *s, float a, float b) {
    volatile float p = a * b;
    s->error += fmaf(a, b, -p);
    tsum_add(s, p);
}
static inline float tsum_total(tsum s) { return s.value + s.error; }

#endif
