#include "nkb_world.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace nkb {

namespace {

constexpr uint32_t kMaxStepsPerLaunch = 64u;
constexpr uint32_t kTreeCrossoverPairs = 4096u;   // admissible pairs above which the tree broadphase is the default
constexpr int kOk = 0, kInvalidArg = 1, kCudaError = 3, kParseError = 5, kOutOfMemory = 6, kNotSupported = 7;

struct BlobEntry { uint32_t dtype; uint64_t n; const uint8_t* data; };

bool BlobFind(const uint8_t* blob, size_t bytes, const char* name, BlobEntry* out) {
    if (bytes < 8 || std::memcmp(blob, "NKT1", 4) != 0) return false;
    uint32_t count;
    std::memcpy(&count, blob + 4, 4);
    size_t at = 8;
    for (uint32_t i = 0; i < count; ++i) {
        if (at + 48 > bytes) return false;
        uint32_t dtype; uint64_t n;
        std::memcpy(&dtype, blob + at + 32, 4);
        std::memcpy(&n, blob + at + 40, 8);
        if (dtype > 3u || n > (uint64_t{1} << 40)) return false;
        const size_t esz = dtype == 3u ? 8u : 4u;
        const size_t payload = static_cast<size_t>((n * esz + 7u) & ~uint64_t{7});
        if (payload > bytes - at - 48) return false;
        if (std::strncmp(reinterpret_cast<const char*>(blob + at), name, 32) == 0) { *out = {dtype, n, blob + at + 48}; return true; }
        at += 48 + payload;
    }
    return false;
}

// dtype code of a record (0 f32, 1 u32, 2 i32, 3 u64) that a vector of T may be filled from
// Walks every record header once: a container whose directory does not fit its byte count is rejected as a whole, so
// a cut-off optional record cannot pass for an absent one.
void BlobValidate(const uint8_t* blob, size_t bytes) {
    uint32_t count;
    std::memcpy(&count, blob + 4, 4);
    size_t at = 8;
    for (uint32_t i = 0; i < count; ++i) {
        if (bytes < 48 || at > bytes - 48) throw Error(kParseError, "template container is truncated");
        uint32_t dtype; uint64_t n;
        std::memcpy(&dtype, blob + at + 32, 4);
        std::memcpy(&n, blob + at + 40, 8);
        if (dtype > 3u) throw Error(kParseError, "template record has an unknown dtype");
        if (n > (uint64_t{1} << 40)) throw Error(kParseError, "template record count exceeds the container");
        const size_t payload = static_cast<size_t>((n * (dtype == 3u ? 8u : 4u) + 7u) & ~uint64_t{7});
        if (payload > bytes - at - 48) throw Error(kParseError, "template record exceeds the container");
        at += 48 + payload;
    }
}

template <typename T> constexpr uint32_t DtypeOf();
template <> constexpr uint32_t DtypeOf<float>() { return 0u; }
template <> constexpr uint32_t DtypeOf<uint32_t>() { return 1u; }
template <> constexpr uint32_t DtypeOf<int32_t>() { return 2u; }
template <> constexpr uint32_t DtypeOf<unsigned long long>() { return 3u; }

// The blob is untrusted: a record is only copied when its dtype is the one the field is read as, so the byte count
// BlobFind bounds-checked (n x the dtype's element size) is the byte count copied.
template <typename T>
std::vector<T> BlobVec(const uint8_t* blob, size_t bytes, const char* name, uint64_t expect) {
    BlobEntry e;
    if (!BlobFind(blob, bytes, name, &e)) throw Error(kParseError, std::string("template field missing or truncated: ") + name);
    if (e.dtype != DtypeOf<T>()) throw Error(kParseError, std::string("template field has the wrong dtype: ") + name);
    if (e.n != expect) throw Error(kParseError, std::string("template field has the wrong size: ") + name);
    std::vector<T> v(static_cast<size_t>(e.n));
    if (e.n) std::memcpy(v.data(), e.data, static_cast<size_t>(e.n) * sizeof(T));
    return v;
}

uint32_t JointDofs(uint32_t t) { return (t == kRevolute || t == kPrismatic) ? 1u : t == kFloating ? 6u : t == kSpherical ? 3u : 0u; }

// ShapeFilterAdmits, reference src/collision/shape_kind.hpp:26-33
bool FilterAdmits(uint32_t ta, uint32_t aa, uint32_t ga_, uint32_t tb, uint32_t ab, uint32_t gb_) {
    if (((ta & ab) | (tb & aa)) == 0u) return false;
    const int32_t ga = static_cast<int32_t>(ga_), gb = static_cast<int32_t>(gb_);
    return !(ga != 0 && gb != 0 && (ga > 0 ? (ga != gb && gb > 0) : ga == gb));
}

}  // namespace

HostTemplate HostTemplate::Parse(const void* blob_in, size_t bytes) {
    const auto* blob = static_cast<const uint8_t*>(blob_in);
    if (blob == nullptr || bytes < 8 || std::memcmp(blob, "NKT1", 4) != 0) throw Error(kParseError, "not a cooked template (NKT1) blob");
    BlobValidate(blob, bytes);
    HostTemplate t;
    const auto cf = BlobVec<float>(blob, bytes, "cfg_f", 10);
    const auto cu = BlobVec<uint32_t>(blob, bytes, "cfg_u", 6);
    t.cfg.dt = cf[0]; t.cfg.gravity[0] = cf[1]; t.cfg.gravity[1] = cf[2]; t.cfg.gravity[2] = cf[3];
    t.cfg.pos_beta = cf[4]; t.cfg.pos_slop = cf[5]; t.cfg.contact_margin = cf[6];
    t.cfg.baumgarte_max_velocity = cf[7]; t.cfg.overlap_recovery_velocity = cf[8]; t.cfg.velocity_tolerance = cf[9];
    t.cfg.vel_iters = cu[0]; t.cfg.pos_iters = cu[1]; t.cfg.max_contacts = cu[2]; t.cfg.max_pairs = cu[3];
    t.cfg.control_mode = 0u;       // the world descriptor selects another mode
    t.cfg.task_link = 0u;
    // sweep counts bound the length of one kernel launch, which cannot be cancelled once it runs
    if (t.cfg.vel_iters > 65535u || t.cfg.pos_iters > 65535u) throw Error(kInvalidArg, "template iteration counts must not exceed 65535");
    t.L = cu[4]; t.B = cu[5];
    const uint32_t L = t.L, B = t.B;
    if (L > kMaxLinks) throw Error(kNotSupported, "more than 32 links per env");
    if (B > kMaxBodies) throw Error(kNotSupported, "more than 256 collidable rows per env");
    if (t.cfg.max_contacts > 1024u) throw Error(kNotSupported, "more than 1024 contact slots per env");
    t.parent = BlobVec<uint32_t>(blob, bytes, "parent", L);
    t.jtype = BlobVec<uint32_t>(blob, bytes, "jtype", L);
    t.link_body = BlobVec<uint32_t>(blob, bytes, "link_body", L);
    t.geom_kind = BlobVec<uint32_t>(blob, bytes, "geom_kind", L);
    t.limit_flags = BlobVec<uint32_t>(blob, bytes, "limit_flags", L);
    t.axis = BlobVec<float>(blob, bytes, "axis", 3 * L);
    const auto local_pos = BlobVec<float>(blob, bytes, "local_pos", 3 * L);
    t.local_quat = BlobVec<float>(blob, bytes, "local_quat", 4 * L);
    const auto parent_offset = BlobVec<float>(blob, bytes, "parent_offset", 3 * L);
    const auto inertia = BlobVec<float>(blob, bytes, "inertia", 36 * L);
    t.damping = BlobVec<float>(blob, bytes, "damping", L);
    t.armature = BlobVec<float>(blob, bytes, "armature", L);
    t.frictionloss = BlobVec<float>(blob, bytes, "frictionloss", L);
    t.stiffness = BlobVec<float>(blob, bytes, "stiffness", L);
    t.spring_ref = BlobVec<float>(blob, bytes, "spring_ref", L);
    t.limit_lower = BlobVec<float>(blob, bytes, "limit_lower", L);
    t.limit_upper = BlobVec<float>(blob, bytes, "limit_upper", L);
    t.geom_pos = BlobVec<float>(blob, bytes, "geom_pos", 3 * L);
    t.geom_quat = BlobVec<float>(blob, bytes, "geom_quat", 4 * L);
    {   // shape frames per collidable row: the template's own, or each link's single shape frame (filled below)
        BlobEntry gk;
        if (BlobFind(blob, bytes, "body_geom_kind", &gk)) {
            t.body_geom_kind = BlobVec<uint32_t>(blob, bytes, "body_geom_kind", B);
            t.body_geom_pos = BlobVec<float>(blob, bytes, "body_geom_pos", 3 * B);
            t.body_geom_quat = BlobVec<float>(blob, bytes, "body_geom_quat", 4 * B);
        }
    }
    {   // optional capacity: contact points per env that get solver rows
        BlobEntry mp;
        t.max_points = 0u;
        if (BlobFind(blob, bytes, "max_points", &mp)) {
            t.max_points = BlobVec<uint32_t>(blob, bytes, "max_points", 1)[0];
            if (t.max_points > 1024u) throw Error(kInvalidArg, "max_points above 1024");
        }
        BlobEntry names;
        if (BlobFind(blob, bytes, "link_names", &names)) {
            // NUL-terminated names in link order inside a word array; exactly L of them, the rest padding
            if (names.dtype != 1u) throw Error(kParseError, "link_names must be a u32 record");
            const char* text = reinterpret_cast<const char*>(names.data);
            const size_t length = static_cast<size_t>(names.n) * 4u;
            size_t at = 0;
            for (uint32_t l = 0; l < L; ++l) {
                const void* end = at < length ? std::memchr(text + at, 0, length - at) : nullptr;
                if (end == nullptr) throw Error(kParseError, "link_names holds fewer names than links");
                const size_t stop = static_cast<size_t>(static_cast<const char*>(end) - text);
                t.link_names.emplace_back(text + at, stop - at);
                at = stop + 1u;
            }
        }
    }
    t.q0 = BlobVec<float>(blob, bytes, "q0", L);
    t.base_pose0 = BlobVec<float>(blob, bytes, "base_pose0", 7);
    t.kp0 = BlobVec<float>(blob, bytes, "kp0", L);
    t.kd0 = BlobVec<float>(blob, bytes, "kd0", L);
    t.force_limit0 = BlobVec<float>(blob, bytes, "force_limit0", L);
    t.shape_kind = BlobVec<uint32_t>(blob, bytes, "shape_kind", B);
    t.contype = BlobVec<uint32_t>(blob, bytes, "contype", B);
    t.conaffinity = BlobVec<uint32_t>(blob, bytes, "conaffinity", B);
    t.group = BlobVec<uint32_t>(blob, bytes, "group", B);
    t.body_to_link = BlobVec<uint32_t>(blob, bytes, "body_to_link", B);
    t.body_id = BlobVec<int32_t>(blob, bytes, "body_id", B);
    t.shape_params = BlobVec<float>(blob, bytes, "shape_params", 4 * B);
    t.mu = BlobVec<float>(blob, bytes, "mu", B);
    t.inv_mass = BlobVec<float>(blob, bytes, "inv_mass", B);
    t.inv_inertia = BlobVec<float>(blob, bytes, "inv_inertia", 3 * B);
    t.inertial_pos = BlobVec<float>(blob, bytes, "inertial_pos", 3 * B);
    t.inertial_quat = BlobVec<float>(blob, bytes, "inertial_quat", 4 * B);
    t.body_pose0 = BlobVec<float>(blob, bytes, "body_pose0", 7 * B);
    BlobEntry ex;
    if (BlobFind(blob, bytes, "excluded", &ex) && ex.n) {
        t.excluded = BlobVec<unsigned long long>(blob, bytes, "excluded", ex.n);
        if (!std::is_sorted(t.excluded.begin(), t.excluded.end())) throw Error(kParseError, "excluded pair keys must ascend");
    }
    // derived tree tables
    t.depth.assign(L, 0); t.link_dof.assign(L, 0); t.anc_mask.assign(L, 0); t.offset.assign(3 * L, 0.f);
    for (uint32_t l = 0; l < L; ++l) {
        const uint32_t p = t.parent[l];
        if (p != kNoLink && p >= l) throw Error(kParseError, "links must follow their parents");
        if (p == kNoLink && l != 0u) throw Error(kNotSupported, "one articulation (a single root link) per env");
        if (t.jtype[l] == kSpherical) throw Error(kNotSupported, "spherical joints");
        if (t.jtype[l] > kSpherical) throw Error(kParseError, "unknown joint type");
        if (t.jtype[l] == kFloating && p != kNoLink) throw Error(kParseError, "a floating joint must be the root");
        t.depth[l] = p == kNoLink ? 0u : t.depth[p] + 1u;
        t.max_depth = std::max(t.max_depth, t.depth[l]);
        t.link_dof[l] = t.ndof;
        for (uint32_t c = 0; c < JointDofs(t.jtype[l]); ++c) t.dof_link.push_back(l);
        t.ndof += JointDofs(t.jtype[l]);
        t.anc_mask[l] = (p == kNoLink ? 0u : t.anc_mask[p]) | (1u << l);
        for (int k = 0; k < 3; ++k) t.offset[3 * l + k] = local_pos[3 * l + k] + parent_offset[3 * l + k];
        if (t.link_body[l] >= B && B != 0u) throw Error(kParseError, "link_body out of range");
        if (t.limit_flags[l] > 3u) throw Error(kParseError, "limit_flags holds bits beyond lower | upper");
        if (t.geom_kind[l] > 1u) throw Error(kParseError, "geom_kind must be 0 (shape frame = link frame) or 1 (own frame)");
    }
    if (t.ndof > kMaxDof) throw Error(kNotSupported, "more than 64 articulation coordinates per env");
    t.floating_root = (L > 0 && t.jtype[0] == kFloating) ? 1u : 0u;
    t.child_begin.assign(L + 1, 0);
    for (uint32_t l = 0; l < L; ++l) {
        t.child_begin[l] = static_cast<uint32_t>(t.children.size());
        for (uint32_t c = 0; c < L; ++c) if (t.parent[c] == l) t.children.push_back(c);
    }
    t.child_begin[L] = static_cast<uint32_t>(t.children.size());
    if (t.children.empty()) t.children.push_back(0);
    // rigid-body form of the 6x6 link inertias: [[I, h^x], [-h^x, m 1]]
    t.inertia10.assign(10 * L, 0.f);
    for (uint32_t l = 0; l < L; ++l) {
        const float* I = inertia.data() + 36 * l;
        const float m = I[3 * 6 + 3];
        const float hx = I[2 * 6 + 4], hy = I[0 * 6 + 5], hz = I[1 * 6 + 3];
        float* o = t.inertia10.data() + 10 * l;
        o[0] = m; o[1] = hx; o[2] = hy; o[3] = hz;
        o[4] = I[0]; o[5] = I[7]; o[6] = I[14]; o[7] = I[1]; o[8] = I[2]; o[9] = I[8];
        // verify the structure so a non-rigid-body matrix is rejected rather than silently reshaped
        const float ref[36] = {o[4], o[7], o[8], 0.f, -hz, hy,   o[7], o[5], o[9], hz, 0.f, -hx,   o[8], o[9], o[6], -hy, hx, 0.f,
                               0.f, hz, -hy, m, 0.f, 0.f,   -hz, 0.f, hx, 0.f, m, 0.f,   hy, -hx, 0.f, 0.f, 0.f, m};
        float scale = 1e-6f;
        for (int k = 0; k < 36; ++k) scale = std::max(scale, std::fabs(I[k]));
        for (int k = 0; k < 36; ++k)
            if (std::fabs(I[k] - ref[k]) > 1e-5f * scale) throw Error(kNotSupported, "link spatial inertia is not of rigid-body form");
    }
    // admissible body-row pairs
    const bool own_frames = !t.body_geom_kind.empty() || B == 0u;
    if (!own_frames) { t.body_geom_kind.assign(B, 0u); t.body_geom_pos.assign(3u * B, 0.f); t.body_geom_quat.assign(4u * B, 0.f); }
    for (uint32_t b = 0; b < B; ++b) {
        if (t.body_to_link[b] != kNoLink && t.body_to_link[b] >= L) throw Error(kParseError, "body_to_link out of range");
        if (!own_frames) {
            const uint32_t l = t.body_to_link[b];
            t.body_geom_quat[4u * b] = 1.f;
            if (l != kNoLink) {
                t.body_geom_kind[b] = t.geom_kind[l];
                for (int k = 0; k < 3; ++k) t.body_geom_pos[3u * b + k] = t.geom_pos[3u * l + k];
                for (int k = 0; k < 4; ++k) t.body_geom_quat[4u * b + k] = t.geom_quat[4u * l + k];
            }
        }
        if (t.shape_kind[b] > kPlane && t.shape_kind[b] != kCylinder) throw Error(kNotSupported, "shape kind without an analytic manifold");
        if (t.body_geom_kind[b] > 1u) throw Error(kParseError, "body_geom_kind must be 0 or 1");
    }
    t.adm_mask.assign(std::max<size_t>(1, static_cast<size_t>(B) * ((B + 31u) / 32u)), 0u);
    for (uint32_t a = 0; a < B; ++a) for (uint32_t b = a + 1; b < B; ++b) {
        if (t.body_id[a] < 0 && t.body_id[b] < 0) continue;
        if (!FilterAdmits(t.contype[a], t.conaffinity[a], t.group[a], t.contype[b], t.conaffinity[b], t.group[b])) continue;
        const unsigned long long key = (static_cast<unsigned long long>(a) << 32) | b;
        if (std::binary_search(t.excluded.begin(), t.excluded.end(), key)) continue;
        const uint32_t ka = t.shape_kind[a], kb = t.shape_kind[b];
        // analytic manifolds exist for a cylinder against a plane or a sphere only (analytical_manifold.hpp:948-949)
        const bool cylinder_other = (ka == kCylinder && kb != kPlane && kb != kSphere) || (kb == kCylinder && ka != kPlane && ka != kSphere);
        const bool analytic = !((ka == kCapsule && kb == kBox) || (ka == kBox && kb == kCapsule) || (ka == kPlane && kb == kPlane) || cylinder_other);
        if (!analytic) throw Error(kNotSupported, "capsule-box pairs and cylinders against anything but planes and spheres need the convex narrowphase, which this path does not provide");
        t.adm_pairs.push_back((a << 16) | b);
        t.adm_mask[a * ((B + 31u) / 32u) + (b >> 5)] |= 1u << (b & 31u);
    }
    if (t.adm_pairs.empty()) t.adm_pairs.push_back(0);
    // free dynamic bodies get their own slot in the rigid-block arrays; every other row shares one scratch slot
    t.free_slot.assign(std::max(B, 1u), 0u);
    t.n_free = 0;
    for (uint32_t b = 0; b < B; ++b) if (t.inv_mass[b] > 0.f && t.body_to_link[b] == kNoLink) ++t.n_free;
    {
        uint32_t next = 0;
        for (uint32_t b = 0; b < B; ++b) t.free_slot[b] = (t.inv_mass[b] > 0.f && t.body_to_link[b] == kNoLink) ? next++ : t.n_free;
    }
    t.joint_rows = 0;
    for (uint32_t l = 0; l < L; ++l) {
        if (JointDofs(t.jtype[l]) != 1u) continue;
        t.joint_rows += ((t.limit_flags[l] & 1u) ? 1u : 0u) + ((t.limit_flags[l] & 2u) ? 1u : 0u) + (t.frictionloss[l] > 0.f ? 1u : 0u) + 1u;
    }
    if (!(t.cfg.dt > 0.f) || !std::isfinite(t.cfg.dt)) throw Error(kInvalidArg, "template dt must be positive");
    return t;
}

void World::Check(cudaError_t err, const char* what) {
    if (err == cudaSuccess) return;
    const int code = err == cudaErrorMemoryAllocation ? kOutOfMemory : kCudaError;
    throw Error(code, std::string(what) + ": " + cudaGetErrorString(err));
}

template <typename T>
T* World::Alloc(size_t count, bool zero) {
    void* p = nullptr;
    const size_t bytes = std::max<size_t>(count, 1) * sizeof(T);
    Check(cudaMalloc(&p, bytes), "cudaMalloc");
    allocations_.push_back(p);
    if (zero) Check(cudaMemsetAsync(p, 0, bytes, stream_), "cudaMemset");
    return static_cast<T*>(p);
}

template <typename T>
const T* World::Upload(const std::vector<T>& v) {
    T* p = Alloc<T>(v.size(), v.empty());
    if (!v.empty()) Check(cudaMemcpyAsync(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice, stream_), "template upload");
    return p;
}

void World::BuildLayout() {
    const HostTemplate& t = tpl_;
    SmemLayout& s = params_.sm;
    const uint32_t L = t.L, B = t.B, n = t.ndof, S = t.cfg.max_contacts;
    TemplateView& tv = params_.t;
    // contact points the admissible pairs can produce in the S slots: sphere pairs give 1 point, capsule pairs 2,
    // box/plane pairs up to 4; the S largest capacities bound what one step can hold
    {
        std::vector<uint32_t> caps;
        if (!(t.adm_pairs.size() == 1 && t.adm_pairs[0] == 0u))
            for (uint32_t key : t.adm_pairs) {
                const uint32_t ka = t.shape_kind[key >> 16], kb = t.shape_kind[key & 0xffffu];
                caps.push_back((ka == kSphere || kb == kSphere) ? 1u : (ka == kCapsule || kb == kCapsule) ? 2u : 4u);      // a cylinder on a plane: up to 4
            }
        std::sort(caps.begin(), caps.end(), [](uint32_t a, uint32_t b) { return a > b; });
        uint32_t total = 0;
        for (size_t k = 0; k < caps.size() && k < S; ++k) total += caps[k];
        // bounds the head records and Jacobian pool in shared memory; the template may ask for more than the default
        tv.point_cap = std::min(total, t.max_points != 0u ? t.max_points : 128u);
    }
    tv.head_cap = (tv.point_cap + t.joint_rows + 3u) & ~3u;
    if (tv.head_cap == 0u) tv.head_cap = 4u;
    if (t.cfg.control_mode == 4u) {
        // the operational-space controller keeps its matrices in the head records' region between the two dynamics passes
        if (t.cfg.task_link >= L) throw Error(kInvalidArg, "osc_task_link is not a link of the articulation");
        const uint32_t need = n * n + 8u * n + 14u * n + 140u;
        if (kHeadStride * tv.head_cap < need) tv.head_cap = ((need + kHeadStride - 1u) / kHeadStride + 3u) & ~3u;
    }
    uint32_t at = 0;
    auto take = [&](uint32_t words) { const uint32_t o = at; at += (words + 3u) & ~3u; return o; };     // 16-byte aligned regions
    // float4-readable matrix rows: a multiple of 4 words that is 4 mod 8 (conflict-free for one lane per row)
    auto pad_ld = [](uint32_t k) { const uint32_t ld = (k + 3u) & ~3u; return (ld & 7u) == 0u ? ld + 4u : ld; };
    s.ld = pad_ld(n);
    s.pose = take(7 * L); s.vel = take(6 * L);
    // the dynamics stage's link scratch and the solver's Newton scratch are live at different times and share one region
    const uint32_t hn = std::max(n, 6u);
    const uint32_t overlay = at;
    s.xrot = take(9 * L); s.xtr = take(3 * L); s.vbias = 0; s.acc = take(6 * L); s.pbias = take(6 * L); s.ic = take(10 * L);
    const uint32_t dynamics_end = at;
    if (std::getenv("NUKA_B200_NO_OVERLAY") == nullptr) at = overlay;
    s.chol = take(hn * pad_ld(hn)); s.bm6 = take(72 + 24);
    s.rjac_heads = t.n_free ? std::min(tv.head_cap, 32u) : 0u;
    s.rjac = take(24 * s.rjac_heads);
    at = std::max(at, dynamics_end);
    s.mass = take(n * s.ld); s.factor = take(n * s.ld); s.vstride = n > 32u ? 64u : 32u;
    s.vecs = take(6 * s.vstride);
    const uint32_t slots = B ? t.n_free + 1u : 0u;
    s.bpose = take(7 * B); s.bvel = take(6 * slots);
    s.bwinv = take(6 * slots); s.bmass = take(7 * slots); s.bfree = take(6 * slots); s.bpseudo = take(6 * slots);
    tv.slot_cap = std::min<uint32_t>(S, (t.adm_pairs.size() == 1 && t.adm_pairs[0] == 0u) ? 0u : static_cast<uint32_t>(t.adm_pairs.size()));
    const uint32_t SC = tv.slot_cap;
    s.pairs = take(SC); s.ccount = take(SC); s.cpoint = take(12 * SC); s.cnormal = take(12 * SC); s.cdepth = take(4 * SC);
    s.cfeat = take(8 * SC);                       // contact identity words
    // before the heads exist the region serves the tree broadphase and then the narrowphase as scratch
    s.heads = take(std::max(kHeadStride * tv.head_cap, SC != 0u ? std::max(lbvh_scratch_words(B), manifold_scratch_words(B, t.n_free != 0u ? kWarpsPerBlockMax : 1u)) : 0u));
    // the Jacobian pool also holds the AABBs (dead once the narrowphase is done) and, after the solve, the cache staging
    // entries + owner marks
    const uint32_t stage_cap = std::min(tv.point_cap, 4u * SC);
    s.jpool = take(std::max(std::max(tv.point_cap * 3u * ((n + 3u) & ~3u), stage_cap * 10u + 4u * SC), 6u * B));
    s.cstage = s.jpool; s.aabb = s.jpool;
    const uint32_t nb = B + (n ? 1u : 0u);
    s.binfo = take(3 * nb + 1 + 2 * tv.head_cap + 2 * s.vstride + nb + 1);      // the unit-row table holds 16-bit head indices
    if (const char* pad = std::getenv("NUKA_B200_SMEM_PAD_WORDS")) at += (static_cast<uint32_t>(std::atoi(pad)) + 3u) & ~3u;   // occupancy experiments
    // Team mode.  An env of many free bodies fills most of an SM's shared memory by itself, so one warp per env would
    // leave the SM with one or two resident warps; instead several warps share the env and descend the rigid blocks
    // of one colour side by side (blocks of a colour share no constraint row).  Registers allow about 11 resident
    // warps per SM, so teams only pay where shared memory already holds residency below that.
    s.team = 1u; s.team_area = at; s.helper_words = 0u; s.team_drill = 0u;
    if (const char* drill = std::getenv("NUKA_B200_TEAM_DRILL")) s.team_drill = static_cast<uint32_t>(std::atoi(drill)) & 3u;
    {
        const uint32_t helper = (s.rjac + 24u * s.rjac_heads - s.chol) + 6u * s.vstride;     // Newton matrix, block mass, staged rows as the env lays them out; vectors
        uint32_t team = 1u;
        if (t.n_free >= 8u) {
            const uint32_t envs_alone = std::max<uint32_t>(1u, (227u * 1024u) / (at * 4u + 1024u));      // resident envs, one warp each
            while (team * 2u <= kWarpsPerBlockMax && envs_alone * team * 2u <= 11u &&
                   (at + 12u + 4u * (team * 2u) + helper * (team * 2u - 1u)) * 4u <= 220u * 1024u) team *= 2u;
        }
        if (const char* forced = std::getenv("NUKA_B200_TEAM")) {                        // team-size experiments
            const uint32_t w = static_cast<uint32_t>(std::atoi(forced));
            if (w >= 1u && w <= kWarpsPerBlockMax && t.n_free != 0u && (at + 12u + 4u * w + helper * (w - 1u)) * 4u <= 220u * 1024u) team = w;
        }
        if (team > 1u) {
            s.team = team; s.helper_words = (helper + 3u) & ~3u;
            s.team_area = take(12u + ((4u * team + 3u) & ~3u) + s.helper_words * (team - 1u));
        }
    }
    s.words = at;
    const size_t bytes = static_cast<size_t>(s.words) * 4u;
    if (bytes > 220u * 1024u) throw Error(kNotSupported, "template needs more shared memory per env than one SM provides");
    // kernel build (regular or slim) and block shape: what keeps the most warps resident on one SM
    const uint32_t team = s.team;                  // a block holds whole teams: w counts warps, w / team envs
    size_t resident[2][kWarpsPerBlockMax + 1] = {{0}, {0}};
    size_t best[2] = {0, 0};
    const bool control = t.cfg.control_mode == 3u || t.cfg.control_mode == 4u;       // these modes run the kernel builds that hold the controllers
    const bool has_slim = step_kernel_has_slim(n, t.n_free, control);
    for (int slim = 0; slim < (has_slim ? 2 : 1); ++slim)
        for (uint32_t w = team; w <= kWarpsPerBlockMax; w += team) {
            if ((w / team) * bytes > 227u * 1024u) break;
            resident[slim][w] = static_cast<size_t>(step_kernel_resident_blocks(n, t.n_free, slim != 0, control, w, (w / team) * bytes)) * w;      // asks the runtime
            best[slim] = std::max(best[slim], resident[slim][w]);
        }
    // The slim build pays about 200 bytes of spills for a fourth warp per scheduler partition: worth it where shared
    // memory lets the extra warps in (measured on the 4096-env quadruped: 15 instead of 12 resident envs per SM, 0.445 ms
    // per step instead of 0.508), not where shared memory caps residency first.
    slim_ = has_slim && best[1] * 10u >= best[0] * 12u;
    if (const char* forced = std::getenv("NUKA_B200_SLIM")) slim_ = has_slim && std::atoi(forced) != 0;     // variant experiments and tests
    const size_t* fits = resident[slim_ ? 1 : 0];
    const size_t most = best[slim_ ? 1 : 0];
    // Block shape: the one that keeps the most warps resident (228 KB shared memory, 1 KB reserved per block); among
    // equals a multiple of 4 warps (one per scheduler, measured 0.5 % faster than 6-warp blocks at the same residency on
    // the quadruped), else the largest.
    warps_per_block_ = team;
    for (uint32_t w = team; w <= kWarpsPerBlockMax; w += team) if (fits[w] == most) warps_per_block_ = w;
    for (uint32_t w = 4; w <= kWarpsPerBlockMax; w += 4) if (w % team == 0u && fits[w] == most) warps_per_block_ = w;
    if (const char* forced = std::getenv("NUKA_B200_WARPS_PER_BLOCK")) {          // block-shape experiments
        const uint32_t w = static_cast<uint32_t>(std::atoi(forced));
        if (w >= 1u && w <= kWarpsPerBlockMax && w % team == 0u && fits[w] != 0u) warps_per_block_ = w;
    }
    if (std::getenv("NUKA_B200_DEBUG_LAYOUT") != nullptr) {
        std::fprintf(stderr, "[nuka_b200] %zu B of shared memory per env, %d registers per thread%s; resident warps per SM by block size:", bytes,
                     step_kernel_registers(n, t.n_free, slim_, control), slim_ ? " (slim build)" : "");
        for (uint32_t w = 1; w <= kWarpsPerBlockMax; ++w) std::fprintf(stderr, " %u:%zu", w, fits[w]);
        std::fprintf(stderr, " -> %u warps per block, %u per env\n", warps_per_block_, team);
        std::fprintf(stderr, "[nuka_b200] word offsets: overlay %u mass %u vecs %u bodies %u contacts %u heads %u pool %u blocks %u end %u\n",
                     s.xrot, s.mass, s.vecs, s.bpose, s.pairs, s.heads, s.jpool, s.binfo, s.words);
    }
}

World::World(int device, cudaStream_t stream, const HostTemplate& tpl, uint32_t env_count)
    : device_(device), stream_(stream), tpl_(tpl), env_count_(env_count) {
    Check(cudaSetDevice(device_), "cudaSetDevice");
    try {
        const HostTemplate& t = tpl_;
        TemplateView& v = params_.t;
        v.L = t.L; v.B = t.B; v.ndof = t.ndof; v.max_depth = t.max_depth; v.floating_root = t.floating_root;
        v.n_excluded = static_cast<uint32_t>(t.excluded.size());
        v.cfg = t.cfg;
        BuildLayout();
        v.parent = Upload(t.parent); v.jtype = Upload(t.jtype); v.depth = Upload(t.depth); v.child_begin = Upload(t.child_begin);
        v.children = Upload(t.children); v.link_dof = Upload(t.link_dof); v.link_body = Upload(t.link_body);
        v.geom_kind = Upload(t.geom_kind); v.limit_flags = Upload(t.limit_flags); v.dof_link = Upload(t.dof_link); v.anc_mask = Upload(t.anc_mask);
        v.axis = Upload(t.axis); v.offset = Upload(t.offset); v.local_quat = Upload(t.local_quat); v.inertia10 = Upload(t.inertia10);
        v.damping = Upload(t.damping); v.armature = Upload(t.armature); v.frictionloss = Upload(t.frictionloss);
        v.stiffness = Upload(t.stiffness); v.spring_ref = Upload(t.spring_ref); v.limit_lower = Upload(t.limit_lower);
        v.limit_upper = Upload(t.limit_upper); v.geom_pos = Upload(t.geom_pos); v.geom_quat = Upload(t.geom_quat);
        v.body_geom_kind = Upload(t.body_geom_kind); v.body_geom_pos = Upload(t.body_geom_pos); v.body_geom_quat = Upload(t.body_geom_quat);
        v.shape_kind = Upload(t.shape_kind); v.contype = Upload(t.contype); v.conaffinity = Upload(t.conaffinity); v.group = Upload(t.group);
        v.body_to_link = Upload(t.body_to_link); v.body_id = Upload(t.body_id); v.shape_params = Upload(t.shape_params); v.mu = Upload(t.mu);
        v.inv_mass = Upload(t.inv_mass); v.inv_inertia = Upload(t.inv_inertia); v.inertial_pos = Upload(t.inertial_pos);
        v.inertial_quat = Upload(t.inertial_quat); v.excluded = Upload(t.excluded);
        v.adm_pairs = Upload(t.adm_pairs);
        v.adm_mask = Upload(t.adm_mask);
        v.free_slot = Upload(t.free_slot); v.n_free = t.n_free;
        v.n_adm = (t.adm_pairs.size() == 1 && t.adm_pairs[0] == 0u) ? 0u : static_cast<uint32_t>(t.adm_pairs.size());
        SetBroadphase(0u);
        const size_t E = env_count_, L = t.L, B = t.B, n = t.ndof, S = t.cfg.max_contacts;
        StateView& s = params_.s;
        s.env_count = env_count_;
        s.q = Alloc<float>(E * L); s.qdot = Alloc<float>(E * L); s.qddot = Alloc<float>(E * L); s.tau = Alloc<float>(E * L);
        s.actuator = Alloc<float>(E * L);
        s.base_pose = Alloc<float>(E * 7); s.link_pose = Alloc<float>(E * L * 7); s.link_vel = Alloc<float>(E * L * 6);
        s.drive_target = Alloc<float>(E * L); s.vel_target = Alloc<float>(E * L); s.noload_speed = Alloc<float>(E * L); s.acc_target = Alloc<float>(E * L); s.kp = Alloc<float>(E * L); s.kd = Alloc<float>(E * L);
        s.force_limit = Alloc<float>(E * L); s.feedforward = Alloc<float>(E * L);
        s.task_target = Alloc<float>(E * 3); s.task_rotation = Alloc<float>(E * 4); s.task_frame = Alloc<float>(E * 7);
        s.null_kp = Alloc<float>(E); s.null_kd = Alloc<float>(E);
        s.body_pose = Alloc<float>(E * B * 7); s.body_linvel = Alloc<float>(E * B * 3); s.body_angvel = Alloc<float>(E * B * 3);
        s.carry_artic = Alloc<float>(E * n); s.carry_rigid = Alloc<float>(E * B * 6); s.limit_lambda = Alloc<float>(E * L * 2);
        s.cache = Alloc<CacheEntry>(E * S * 4);
        s.status = Alloc<uint32_t>(E); s.solver_residual = Alloc<float>(E * 4); s.solver_sweeps = Alloc<uint32_t>(E);
        s.pair_count = Alloc<uint32_t>(E); s.pairs = Alloc<uint32_t>(E * S * 2); s.contact_count = Alloc<uint32_t>(E * S);
        s.contact_point = Alloc<float>(E * S * 12); s.contact_normal = Alloc<float>(E * S * 12); s.contact_depth = Alloc<float>(E * S * 4);
        s.dbg_mass = nullptr; s.dbg_qdot_pseudo = nullptr; s.dbg_cycles = nullptr;
        Seed();
    } catch (...) {
        for (void* p : allocations_) cudaFree(p);
        allocations_.clear();
        throw;
    }
}

World::~World() {
    cudaSetDevice(device_);
    cudaStreamSynchronize(stream_);
    if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
    if (graph_) cudaGraphDestroy(graph_);
    for (void* p : allocations_) cudaFree(p);
}

// Every env starts from the template (reference src/nk/pipeline/world.cpp:289-654); the same table drives
// per-env resets.
void World::Seed() {
    const HostTemplate& t = tpl_;
    StateView& s = params_.s;
    const uint32_t L = t.L, B = t.B, n = t.ndof, S = t.cfg.max_contacts;
    std::vector<CacheEntry> empty(1);
    std::memset(empty.data(), 0, sizeof(CacheEntry));
    empty[0].pair = 0xffffffffu;
    std::vector<CacheEntry> empties(static_cast<size_t>(std::max(1u, 4u * S)), empty[0]);
    cache_empty_ = const_cast<CacheEntry*>(Upload(empties));
    const float* q0 = Upload(t.q0);
    const float* base0 = Upload(t.base_pose0);
    const float* body0 = Upload(t.body_pose0);
    const float* kp0 = Upload(t.kp0);
    const float* kd0 = Upload(t.kd0);
    const float* fl0 = Upload(t.force_limit0);
    reset_.env_count = env_count_;
    reset_.env_ids = nullptr;
    uint32_t f = 0;
    auto add = [&](void* dst, const void* src, uint32_t words) { if (words) { reset_.fields[f++] = {dst, src, words, 0u, 0u}; persistent_.push_back({dst, words}); } };
    add(s.q, q0, L); add(s.qdot, nullptr, L); add(s.qddot, nullptr, L); add(s.tau, nullptr, L); add(s.actuator, nullptr, L);
    add(s.base_pose, base0, L ? 7u : 0u); add(s.link_vel, nullptr, 6 * L);
    add(s.body_pose, body0, 7 * B); add(s.body_linvel, nullptr, 3 * B); add(s.body_angvel, nullptr, 3 * B);
    add(s.carry_artic, nullptr, n); add(s.carry_rigid, nullptr, 6 * B); add(s.limit_lambda, nullptr, 2 * L);
    add(s.cache, cache_empty_, 4 * S * static_cast<uint32_t>(sizeof(CacheEntry) / 4));
    add(s.status, nullptr, 1); add(s.solver_residual, nullptr, 4); add(s.solver_sweeps, nullptr, 1);
    reset_.field_count = f;
    // drive inputs are seeded once; resets keep them (reference nuka.h:378-379)
    ResetParams seed = reset_;
    auto add_seed = [&](void* dst, const void* src, uint32_t words) { if (words) { seed.fields[seed.field_count++] = {dst, src, words, 0u, 0u}; persistent_.push_back({dst, words}); } };
    add_seed(s.drive_target, q0, L); add_seed(s.kp, kp0, L); add_seed(s.kd, kd0, L); add_seed(s.force_limit, fl0, L);
    add_seed(s.vel_target, nullptr, L); add_seed(s.feedforward, nullptr, L); add_seed(s.noload_speed, nullptr, L);
    add_seed(s.acc_target, nullptr, L);
    // operational-space inputs: no target, no orientation task, the task frame at the link's origin, no posture gains
    const float* frame0 = Upload(std::vector<float>{0.f, 0.f, 0.f, 1.f, 0.f, 0.f, 0.f});
    add_seed(s.task_target, nullptr, L ? 3u : 0u); add_seed(s.task_rotation, nullptr, L ? 4u : 0u); add_seed(s.task_frame, frame0, L ? 7u : 0u);
    add_seed(s.null_kp, nullptr, L ? 1u : 0u); add_seed(s.null_kd, nullptr, L ? 1u : 0u);
    Check(launch_reset(seed, env_count_, stream_), "seed launch");
    ++launches_;
    Refresh();
}

size_t World::PersistentBytes() const {
    size_t words = 0;
    for (const PersistentField& f : persistent_) words += static_cast<size_t>(f.words) * env_count_;
    return words * 4u;
}

uint64_t World::PersistentLayoutHash() const {
    uint64_t h = 1469598103934665603ull;      // FNV-1a over the counts that fix the byte layout
    auto mix = [&](uint64_t v) { for (int k = 0; k < 8; ++k) { h ^= (v >> (8 * k)) & 0xffu; h *= 1099511628211ull; } };
    mix(env_count_); mix(tpl_.L); mix(tpl_.B); mix(tpl_.ndof); mix(tpl_.cfg.max_contacts);
    for (const PersistentField& f : persistent_) mix(f.words);
    return h;
}

void World::DownloadPersistent(uint8_t* out) {
    Check(cudaSetDevice(device_), "cudaSetDevice");
    size_t at = 0;
    for (const PersistentField& f : persistent_) {
        const size_t bytes = static_cast<size_t>(f.words) * env_count_ * 4u;
        Check(cudaMemcpyAsync(out + at, f.ptr, bytes, cudaMemcpyDeviceToHost, stream_), "checkpoint download");
        at += bytes;
    }
    Check(cudaStreamSynchronize(stream_), "checkpoint synchronize");
}

void World::UploadPersistent(const uint8_t* in) {
    Check(cudaSetDevice(device_), "cudaSetDevice");
    size_t at = 0;
    for (const PersistentField& f : persistent_) {
        const size_t bytes = static_cast<size_t>(f.words) * env_count_ * 4u;
        Check(cudaMemcpyAsync(f.ptr, in + at, bytes, cudaMemcpyHostToDevice, stream_), "checkpoint upload");
        at += bytes;
    }
    Refresh();
    Check(cudaStreamSynchronize(stream_), "checkpoint synchronize");     // the caller's bytes may go away after the call
}

// Recomputes the derived poses (link poses, body mirrors) from the coordinates: of every env, of the `count` envs
// listed in the device array `ids`, or of the envs whose word in the device array `mask` is non-zero.
void World::Refresh(const uint32_t* ids, uint32_t count, const uint32_t* mask) {
    StepParams p = params_;
    p.mode = kModeRefresh; p.steps = 1;
    p.sel_ids = ids; p.sel_count = ids != nullptr ? count : 0u; p.sel_mask = mask;
    Check(cudaSetDevice(device_), "cudaSetDevice");
    Check(launch_step(p, warps_per_block_, slim_, stream_), "refresh launch");
    ++launches_;
}

void World::RunStage(uint32_t mode) {
    StateView& s = params_.s;
    const size_t E = env_count_, n = tpl_.ndof;
    if (mode == kModeDynamicsOnly && s.dbg_mass == nullptr) { s.dbg_mass = Alloc<float>(E * n * n); graph_valid_ = false; }
    StepParams p = params_;
    p.mode = mode; p.steps = 1;
    Check(cudaSetDevice(device_), "cudaSetDevice");
    Check(launch_step(p, warps_per_block_, slim_, stream_), "stage launch");
    ++launches_;
}

void World::SetGraphMode(bool on) {
    graph_mode_ = on;
    graph_valid_ = false;
}

void World::Step(uint32_t n) {
    if (n == 0u) return;
    step_count_ += n;
    Check(cudaSetDevice(device_), "cudaSetDevice");
    StepParams p = params_;
    p.mode = kModeStep;
    if (!graph_mode_) {
        // the kernel advances several steps per launch (inputs are constant across them; state goes back to global
        // memory after every step, so the split changes no result); the cap keeps any one launch short
        for (uint32_t done = 0u; done < n; done += kMaxStepsPerLaunch) {
            p.steps = std::min(n - done, kMaxStepsPerLaunch);
            Check(launch_step(p, warps_per_block_, slim_, stream_), "step launch");
            ++launches_;
        }
        return;
    }
    if (!graph_valid_) {
        if (graph_exec_) { cudaGraphExecDestroy(graph_exec_); graph_exec_ = nullptr; }
        if (graph_) { cudaGraphDestroy(graph_); graph_ = nullptr; }
        p.steps = 1;
        // configure the kernel's shared-memory attribute outside the capture
        StepParams warm = params_;
        warm.mode = kModeRefresh; warm.steps = 1;
        Check(launch_step(warm, warps_per_block_, slim_, stream_), "graph warm-up launch");
        ++launches_;
        Check(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal), "begin capture");
        const cudaError_t launched = launch_step(p, warps_per_block_, slim_, stream_);
        const cudaError_t ended = cudaStreamEndCapture(stream_, &graph_);
        Check(launched, "captured step launch");
        Check(ended, "end capture");
        Check(cudaGraphInstantiate(&graph_exec_, graph_, 0), "graph instantiate");
        graph_valid_ = true;
    }
    for (uint32_t k = 0; k < n; ++k) { Check(cudaGraphLaunch(graph_exec_, stream_), "graph launch"); ++launches_; }
}

void World::Reset(const uint32_t* env_ids, uint32_t count) {
    Check(cudaSetDevice(device_), "cudaSetDevice");
    ResetParams r = reset_;
    if (env_ids == nullptr) {
        Check(launch_reset(r, env_count_, stream_), "reset launch");
    } else {
        if (count == 0u) return;
        for (uint32_t k = 0; k < count; ++k) if (env_ids[k] >= env_count_) throw Error(kInvalidArg, "reset_envs: env id out of range");
        std::vector<uint32_t> ids(env_ids, env_ids + count);
        std::sort(ids.begin(), ids.end());
        ids.erase(std::unique(ids.begin(), ids.end()), ids.end());
        if (ids.size() > reset_ids_cap_) {
            reset_ids_ = Alloc<uint32_t>(env_count_, false);
            reset_ids_cap_ = env_count_;
        }
        // the id list must outlive the async copy: synchronise the (rare) partial reset path
        Check(cudaMemcpyAsync(reset_ids_, ids.data(), ids.size() * 4u, cudaMemcpyHostToDevice, stream_), "reset ids upload");
        Check(cudaStreamSynchronize(stream_), "reset ids sync");
        r.env_ids = reset_ids_;
        Check(launch_reset(r, static_cast<uint32_t>(ids.size()), stream_), "reset launch");
        launches_ += 2;
        Refresh(reset_ids_, static_cast<uint32_t>(ids.size()), nullptr);
        return;
    }
    ++launches_;
    Refresh();
}

// Resets the envs whose word in the device array `mask` (env_count words, read on the world's stream) is non-zero.
// Everything stays on the stream: no id list crosses to the host and nothing synchronises, so an episode loop can
// chain step -> termination test -> reset without draining the GPU.
void World::ResetMasked(const uint32_t* mask) {
    Check(cudaSetDevice(device_), "cudaSetDevice");
    ResetParams r = reset_;
    r.env_ids = nullptr; r.env_mask = mask;
    Check(launch_reset(r, env_count_, stream_), "masked reset launch");
    ++launches_;
    Refresh(nullptr, 0u, mask);
}

// Same result as Reset(env_ids, count) with no allocation on the device or the host: ids are validated, sorted and
// de-duplicated in a member array, copied into the module's fixed device array, and the stream is drained before
// returning so the member array can be reused (Reset waits for its id copy in the same way).
void World::ResetStaticIds(const uint32_t* env_ids, uint32_t count) {
    Check(cudaSetDevice(device_), "cudaSetDevice");
    if (count == 0u) return;
    if (count > kStaticResetMaxIds) throw Error(kInvalidArg, "reset_envs_static: more than 4096 env ids in one call");
    for (uint32_t k = 0; k < count; ++k) if (env_ids[k] >= env_count_) throw Error(kInvalidArg, "reset_envs_static: env id out of range");
    std::copy(env_ids, env_ids + count, static_ids_host_);
    std::sort(static_ids_host_, static_ids_host_ + count);
    const uint32_t unique = static_cast<uint32_t>(std::unique(static_ids_host_, static_ids_host_ + count) - static_ids_host_);
    ResetParams r = reset_;
    const uint32_t* device_ids = nullptr;
    Check(launch_reset_static_ids(r, static_ids_host_, unique, device_, stream_, &device_ids), "static-id reset launch");
    ++launches_;
    Refresh(device_ids, unique, nullptr);       // derived poses of the reset envs only; reads the ids still in the array
    Check(cudaStreamSynchronize(stream_), "static-id reset sync");
}

void World::PackObservations(const ObservationParams& o, float* device_out) {
    if (tpl_.L < 2u || !tpl_.floating_root) throw Error(kNotSupported, "observation records need a floating-base articulation");
    Check(cudaSetDevice(device_), "cudaSetDevice");
    Check(launch_pack_observations(params_.s, tpl_.L, o, device_out, stream_), "observation pack launch");
    ++launches_;
}

// Route of the candidate-pair stage.  The table route tests every admissible pair's boxes each step (B^2 / 2 tests at
// worst); the tree route sorts, builds and walks a tree of the env's boxes.  Both give the same list, so the choice is
// a matter of cost: by default the tree takes over once the table is longer than kTreeCrossoverPairs.
void World::SetBroadphase(uint32_t mode) {
    if (mode > 2u) throw Error(kInvalidArg, "broadphase mode must be 0 (by size), 1 (table) or 2 (tree)");
    const uint32_t tree = mode == 2u || (mode == 0u && params_.t.n_adm > kTreeCrossoverPairs) ? 1u : 0u;
    if (tree != params_.t.broadphase_tree) { params_.t.broadphase_tree = tree; graph_valid_ = false; }
}

// Contact read-out arrays (pair list, counts, points, normals, depths) are written every step while enabled; a
// caller that only reads robot state switches them off and saves the stores.
void World::SetContactReadout(bool on) {
    StateView& s = params_.s;
    if (on == (s.pair_count != nullptr)) return;
    if (on) { s.pair_count = readout_.pair_count; s.pairs = readout_.pairs; s.contact_count = readout_.contact_count;
              s.contact_point = readout_.contact_point; s.contact_normal = readout_.contact_normal; s.contact_depth = readout_.contact_depth; }
    else { readout_ = s; s.pair_count = nullptr; }
    graph_valid_ = false;
}

void World::Synchronize() {
    Check(cudaSetDevice(device_), "cudaSetDevice");
    Check(cudaStreamSynchronize(stream_), "stream synchronize");
}

bool World::Field(uint32_t id, FieldInfo* out) {
    StateView& s = params_.s;
    const size_t L = tpl_.L, B = tpl_.B, n = tpl_.ndof, S = tpl_.cfg.max_contacts;
    auto set = [&](void* p, size_t per_env, uint32_t dtype, bool w) { *out = {p, per_env, dtype, w}; return true; };
    switch (id) {
        case 0: return set(s.body_pose, B * 7, 0, true);
        case 1: return set(s.link_pose, L * 7, 0, false);
        case 2: return set(s.q, L, 0, true);
        case 3: return set(s.qdot, L, 0, true);
        case 6: return set(s.drive_target, L, 0, true);
        case 7: return set(s.link_vel, L * 6, 0, true);
        case 8: return set(s.kp, L, 0, true);
        case 9: return set(s.kd, L, 0, true);
        case 10: return set(s.force_limit, L, 0, true);
        case 11: return set(s.base_pose, L ? 7 : 0, 0, true);
        case 12: return set(s.drive_target, L, 0, true);       // TORQUE_INPUT aliases DRIVE_TARGET (nuka.h:587-589)
        case 13: return set(s.vel_target, L, 0, true);
        case 14: return set(s.noload_speed, L, 0, true);
        case 22: return set(s.feedforward, L, 0, true);
        case 56: return set(s.acc_target, L, 0, true);
        case 15: return set(s.task_target, L ? 3 : 0, 0, true);
        case 31: return set(s.task_rotation, L ? 4 : 0, 0, true);
        case 32: return set(s.task_frame, L ? 7 : 0, 0, true);
        case 57: return set(s.null_kp, L ? 1 : 0, 0, true);
        case 58: return set(s.null_kd, L ? 1 : 0, 0, true);
        case 25: return set(s.body_linvel, B * 3, 0, true);
        case 26: return set(s.body_angvel, B * 3, 0, true);
        case 27: return set(s.limit_lambda, L * 2, 0, false);
        case 29: return set(s.actuator, L, 0, false);
        case 39: return set(s.status, 1, 1, true);
        case 109: return set(s.solver_residual, 4, 0, false);
        case 0x10000: return set(s.qddot, L, 0, false);
        case 0x10001:
            // a captured graph holds its own copy of the kernel parameters: a tap allocated after the capture forces
            // a new capture, or the graph would keep stepping with a null tap pointer
            if (s.dbg_mass == nullptr) { s.dbg_mass = Alloc<float>(static_cast<size_t>(env_count_) * n * n); graph_valid_ = false; }
            return set(s.dbg_mass, n * n, 0, false);
        // contact read-outs: while switched off (SetContactReadout) the arrays keep the last values written
        case 0x10002: return set(s.pair_count != nullptr ? s.pair_count : readout_.pair_count, 1, 1, false);
        case 0x10003: return set(s.pairs, S * 2, 1, false);
        case 0x10004: return set(s.contact_count, S, 1, false);
        case 0x10005: return set(s.contact_point, S * 12, 0, false);
        case 0x10006: return set(s.contact_normal, S * 12, 0, false);
        case 0x10007: return set(s.contact_depth, S * 4, 0, false);
        case 0x10008: return set(s.solver_sweeps, 1, 1, false);
        case 0x10009:
            if (s.dbg_qdot_pseudo == nullptr) { s.dbg_qdot_pseudo = Alloc<float>(static_cast<size_t>(env_count_) * n); graph_valid_ = false; }
            return set(s.dbg_qdot_pseudo, n, 0, false);
#ifdef NKB_STAGE_TAPS
        case 0x1000A:      // stage cycle counters accumulate from the first request on; writable so callers can clear them
            if (s.dbg_cycles == nullptr) { s.dbg_cycles = Alloc<uint32_t>(static_cast<size_t>(env_count_) * 32u); graph_valid_ = false; }
            return set(s.dbg_cycles, 32, 1, true);
#endif
        default: return false;
    }
}

}  // namespace nkb
