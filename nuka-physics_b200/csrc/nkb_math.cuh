// Device math for the batched articulated step: 3-vectors, quaternions (wxyz), structured spatial transforms.
// Joint transforms are kept as (E, r) pairs (rotation + translation) and rigid-body inertias as
// (mass, h = m c, I about the frame origin) instead of dense 6x6 matrices; the quantities are the ones the
// reference computes in src/math/cuda_spatial_ops.cuh and ops/articulation.cu:91-171.
#pragma once
#include <cuda_runtime.h>
#include <cfloat>
#include <cstdint>

namespace nkb {

#define NKB_FULL 0xffffffffu
#define NKB_DEV __device__ __forceinline__

struct V3 { float x, y, z; };
struct Q4 { float w, x, y, z; };
struct M3 { float m[9]; };
struct Sym3 { float xx, yy, zz, xy, xz, yz; };

NKB_DEV V3 mk3(float x, float y, float z) { V3 r; r.x = x; r.y = y; r.z = z; return r; }
NKB_DEV V3 ld3(const float* p) { return mk3(p[0], p[1], p[2]); }
NKB_DEV void st3(float* p, V3 a) { p[0] = a.x; p[1] = a.y; p[2] = a.z; }
NKB_DEV V3 operator+(V3 a, V3 b) { return mk3(a.x + b.x, a.y + b.y, a.z + b.z); }
NKB_DEV V3 operator-(V3 a, V3 b) { return mk3(a.x - b.x, a.y - b.y, a.z - b.z); }
NKB_DEV V3 operator-(V3 a) { return mk3(-a.x, -a.y, -a.z); }
NKB_DEV V3 operator*(V3 a, float s) { return mk3(a.x * s, a.y * s, a.z * s); }
NKB_DEV float dot(V3 a, V3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
NKB_DEV V3 cross(V3 a, V3 b) { return mk3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x); }
NKB_DEV float len3(V3 a) { return sqrtf(dot(a, a)); }
NKB_DEV float comp(V3 a, int k) { return k == 0 ? a.x : (k == 1 ? a.y : a.z); }
NKB_DEV void setc(V3& a, int k, float v) { if (k == 0) a.x = v; else if (k == 1) a.y = v; else a.z = v; }

NKB_DEV Q4 mkq(float w, float x, float y, float z) { Q4 q; q.w = w; q.x = x; q.y = y; q.z = z; return q; }
NKB_DEV Q4 ldq(const float* p) { return mkq(p[0], p[1], p[2], p[3]); }
NKB_DEV void stq(float* p, Q4 q) { p[0] = q.w; p[1] = q.x; p[2] = q.y; p[3] = q.z; }
NKB_DEV Q4 qmul(Q4 a, Q4 b) {
    return mkq(a.w * b.w - a.x * b.x - a.y * b.y - a.z * b.z, a.w * b.x + a.x * b.w + a.y * b.z - a.z * b.y,
               a.w * b.y - a.x * b.z + a.y * b.w + a.z * b.x, a.w * b.z + a.x * b.y - a.y * b.x + a.z * b.w);
}
// identity when |q|^2 <= eps
NKB_DEV Q4 qnorm_le(Q4 q, float eps) {
    const float n = q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z;
    if (n <= eps) return mkq(1.f, 0.f, 0.f, 0.f);
    const float i = rsqrtf(n);
    return mkq(q.w * i, q.x * i, q.y * i, q.z * i);
}
// identity when |q|^2 < eps
NKB_DEV Q4 qnorm_lt(Q4 q, float eps) {
    const float n = q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z;
    if (n < eps) return mkq(1.f, 0.f, 0.f, 0.f);
    const float i = rsqrtf(n);
    return mkq(q.w * i, q.x * i, q.y * i, q.z * i);
}
NKB_DEV V3 qrot_raw(Q4 q, V3 v) {
    const V3 qv = mk3(q.x, q.y, q.z);
    const V3 t = cross(qv, v) * 2.0f;
    return v + t * q.w + cross(qv, t);
}
NKB_DEV V3 qrot(Q4 q, V3 v) {
    const float n = q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z;
    if (n > 1.0e-12f) { const float i = rsqrtf(n); q.w *= i; q.x *= i; q.y *= i; q.z *= i; }
    return qrot_raw(q, v);
}
NKB_DEV V3 qrot_inv(Q4 q, V3 v) {
    const float n = q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z;
    if (n > 1.0e-12f) { const float i = rsqrtf(n); q.w *= i; q.x *= i; q.y *= i; q.z *= i; }
    return qrot_raw(mkq(q.w, -q.x, -q.y, -q.z), v);
}

NKB_DEV M3 m3_ident() { M3 r; r.m[0] = 1; r.m[1] = 0; r.m[2] = 0; r.m[3] = 0; r.m[4] = 1; r.m[5] = 0; r.m[6] = 0; r.m[7] = 0; r.m[8] = 1; return r; }
NKB_DEV M3 m3_mul(const M3& a, const M3& b) {
    M3 o;
#pragma unroll
    for (int r = 0; r < 3; ++r)
#pragma unroll
        for (int c = 0; c < 3; ++c) o.m[r * 3 + c] = a.m[r * 3] * b.m[c] + a.m[r * 3 + 1] * b.m[c + 3] + a.m[r * 3 + 2] * b.m[c + 6];
    return o;
}
NKB_DEV M3 m3_from_quat(Q4 q) {
    const float n = q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z;
    if (n <= 1.0e-12f) return m3_ident();
    const float i = rsqrtf(n); q.w *= i; q.x *= i; q.y *= i; q.z *= i;
    const float xx = q.x * q.x, yy = q.y * q.y, zz = q.z * q.z, xy = q.x * q.y, xz = q.x * q.z, yz = q.y * q.z;
    const float wx = q.w * q.x, wy = q.w * q.y, wz = q.w * q.z;
    M3 o;
    o.m[0] = 1.0f - 2.0f * (yy + zz); o.m[1] = 2.0f * (xy - wz); o.m[2] = 2.0f * (xz + wy);
    o.m[3] = 2.0f * (xy + wz); o.m[4] = 1.0f - 2.0f * (xx + zz); o.m[5] = 2.0f * (yz - wx);
    o.m[6] = 2.0f * (xz - wy); o.m[7] = 2.0f * (yz + wx); o.m[8] = 1.0f - 2.0f * (xx + yy);
    return o;
}
// sin and cos of a joint angle: three-term Cody-Waite reduction by pi/2 and the classic single-precision minimax
// polynomials on [-pi/4, pi/4] (1-2 ulp for |x| up to a few thousand radians).  The library sinf/cosf carry a
// large-argument path with a local-memory table that this kernel never needs.
NKB_DEV void sincos_joint(float x, float& s, float& c) {
    const float q = rintf(x * 0.636619772f);
    const int quadrant = (int)q;
    float r = fmaf(q, -1.57079601e+00f, x);
    r = fmaf(q, -3.13916473e-07f, r);
    r = fmaf(q, -5.39030253e-15f, r);
    const float r2 = r * r;
    float sp = fmaf(-1.9515295891e-4f, r2, 8.3321608736e-3f);
    sp = fmaf(sp, r2, -1.6666654611e-1f);
    sp = fmaf(sp * r2, r, r);
    float cp = fmaf(2.443315711809948e-5f, r2, -1.388731625493765e-3f);
    cp = fmaf(cp, r2, 4.166664568298827e-2f);
    cp = fmaf(cp * r2, r2, fmaf(-0.5f, r2, 1.0f));
    const float sv = (quadrant & 1) ? cp : sp, cv = (quadrant & 1) ? sp : cp;
    s = (quadrant & 2) ? -sv : sv;
    c = ((quadrant + 1) & 2) ? -cv : cv;
}
NKB_DEV M3 m3_axis_angle(V3 a, float angle) {
    const float l = dot(a, a);
    if (l <= 1.0e-12f) return m3_ident();
    a = a * rsqrtf(l);
    float s, c;
    sincos_joint(angle, s, c);
    const float t = 1.0f - c;
    M3 o;
    o.m[0] = t * a.x * a.x + c; o.m[1] = t * a.x * a.y - s * a.z; o.m[2] = t * a.x * a.z + s * a.y;
    o.m[3] = t * a.x * a.y + s * a.z; o.m[4] = t * a.y * a.y + c; o.m[5] = t * a.y * a.z - s * a.x;
    o.m[6] = t * a.x * a.z - s * a.y; o.m[7] = t * a.y * a.z + s * a.x; o.m[8] = t * a.z * a.z + c;
    return o;
}
NKB_DEV V3 m3_mulv(const float* E, V3 v) {
    return mk3(E[0] * v.x + E[1] * v.y + E[2] * v.z, E[3] * v.x + E[4] * v.y + E[5] * v.z, E[6] * v.x + E[7] * v.y + E[8] * v.z);
}
NKB_DEV V3 m3_tmulv(const float* E, V3 v) {
    return mk3(E[0] * v.x + E[3] * v.y + E[6] * v.z, E[1] * v.x + E[4] * v.y + E[7] * v.z, E[2] * v.x + E[5] * v.y + E[8] * v.z);
}
NKB_DEV V3 sym_mulv(const float* s, V3 v) {   // xx yy zz xy xz yz
    return mk3(s[0] * v.x + s[3] * v.y + s[4] * v.z, s[3] * v.x + s[1] * v.y + s[5] * v.z, s[4] * v.x + s[5] * v.y + s[2] * v.z);
}

// Motion transform X = [[E, 0], [-E r^x, E]]: (w, v) -> (E w, E (v - r x w)).
NKB_DEV void xf_motion(const float* E, V3 r, V3 w, V3 v, V3& ow, V3& ov) {
    ow = m3_mulv(E, w);
    ov = m3_mulv(E, v - cross(r, w));
}
// Force transpose X^T: (n, f) -> (E^T n + r x E^T f, E^T f).
NKB_DEV void xf_force_t(const float* E, V3 r, V3 n, V3 f, V3& on, V3& of) {
    of = m3_tmulv(E, f);
    on = m3_tmulv(E, n) + cross(r, of);
}
// Rigid-body inertia stored as 10 floats: m, h(3) = m c, I(6) = xx yy zz xy xz yz about the frame origin.
// I v for a motion vector (w, v): (I w + h x v, m v - h x w).
NKB_DEV void rbi_mulv(const float* I10, V3 w, V3 v, V3& on, V3& of) {
    const V3 h = ld3(I10 + 1);
    on = sym_mulv(I10 + 4, w) + cross(h, v);
    of = v * I10[0] - cross(h, w);
}
// X^T I X for a rigid-body inertia: rotate by E^T and shift by r (parallel axis in the parent frame).
NKB_DEV void rbi_to_parent(const float* E, V3 r, const float* I10, float* out) {
    const float m = I10[0];
    const V3 h = m3_tmulv(E, ld3(I10 + 1));            // m c expressed in the parent frame (child origin)
    // I_parent_axes = E^T I E
    const float* s = I10 + 4;
    const float I[9] = {s[0], s[3], s[4], s[3], s[1], s[5], s[4], s[5], s[2]};
    float T[9];
#pragma unroll
    for (int a = 0; a < 3; ++a)
#pragma unroll
        for (int b = 0; b < 3; ++b) T[a * 3 + b] = I[a * 3] * E[b] + I[a * 3 + 1] * E[3 + b] + I[a * 3 + 2] * E[6 + b];
    float R[9];
#pragma unroll
    for (int a = 0; a < 3; ++a)
#pragma unroll
        for (int b = 0; b < 3; ++b) R[a * 3 + b] = E[a] * T[b] + E[3 + a] * T[3 + b] + E[6 + a] * T[6 + b];
    // shift origin by r: h' = h + m r;  I' = I - (h x)(r x) - (r x)(h' x)   [Featherstone: I + r^x h^x^T ...]
    // With c = h/m the child COM from the child origin, the COM from the parent origin is c + r and
    // I' = I_child_origin + m ((c+r).(c+r) 1 - (c+r)(c+r)^T) - m (c.c 1 - c c^T).
    const V3 hp = h + r * m;
    // m (a.a 1 - a a^T) with a = hp/m equals (hp.a) 1 - hp a^T; written with h and r to avoid dividing by m:
    // m(c+r).(c+r) - m c.c = 2 h.r + m r.r ;  m (c+r)(c+r)^T - m c c^T = h r^T + r h^T + m r r^T
    const float d = 2.0f * dot(h, r) + m * dot(r, r);
    out[0] = m;
    out[1] = hp.x; out[2] = hp.y; out[3] = hp.z;
    out[4] = R[0] + d - (2.0f * h.x * r.x + m * r.x * r.x);
    out[5] = R[4] + d - (2.0f * h.y * r.y + m * r.y * r.y);
    out[6] = R[8] + d - (2.0f * h.z * r.z + m * r.z * r.z);
    out[7] = R[1] - (h.x * r.y + r.x * h.y + m * r.x * r.y);
    out[8] = R[2] - (h.x * r.z + r.x * h.z + m * r.x * r.z);
    out[9] = R[5] - (h.y * r.z + r.y * h.z + m * r.y * r.z);
}

// motion cross: (lw, lv) x (rw, rv)
NKB_DEV void motion_cross(V3 lw, V3 lv, V3 rw, V3 rv, V3& ow, V3& ov) { ow = cross(lw, rw); ov = cross(lw, rv) + cross(lv, rw); }
// force cross: (w, v) x* (n, f)
NKB_DEV void force_cross(V3 w, V3 v, V3 n, V3 f, V3& on, V3& of) { on = cross(w, n) + cross(v, f); of = cross(w, f); }

// compensated float sum (value + error), as the reference's TileSum (ops/block_descent_tile.cuh:15-46)
struct CSum { float value, error; };
NKB_DEV void csum_add(CSum& s, float x) {
    const float sum = __fadd_rn(s.value, x);
    const float part = __fsub_rn(sum, s.value);
    s.error += __fadd_rn(__fsub_rn(s.value, __fsub_rn(sum, part)), __fsub_rn(x, part));
    s.value = sum;
}
NKB_DEV void csum_addp(CSum& s, float a, float b) {
    const float p = __fmul_rn(a, b);
    s.error += fmaf(a, b, -p);
    csum_add(s, p);
}
NKB_DEV float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(NKB_FULL, v, o);
    return v;
}
NKB_DEV float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(NKB_FULL, v, o));
    return v;
}
NKB_DEV float warp_csum_total(CSum s) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(NKB_FULL, s.value, o);
        s.error += __shfl_xor_sync(NKB_FULL, s.error, o);
        csum_add(s, v);
    }
    return s.value + s.error;
}

}  // namespace nkb
