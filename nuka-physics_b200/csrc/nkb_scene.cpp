// In-library scene cooker: a `.nks` scene document (the reference's JSON scene format, src/scene/format/nks.cpp) becomes
// the cooked template this library creates worlds from, so that nuka_world_create_from_scene takes the file the
// reference takes.  The rules are those of the reference's cooker for the part this path covers
// (runtime/articulation/articulation_state.cpp:392-426 for the joint frames, src/scene/cook/cook_to_model.cpp for the
// collidable rows, their order, filters and the parent-child exclusions): one tree of rigid bodies joined by revolute /
// prismatic / fixed joints under a free or static root, sphere / capsule / box shapes with local frames (several per
// link), free rigid bodies with one shape each, static ground planes, position actuators as drives.  Everything else in a
// scene (meshes, cylinders, heightfields, sensors, materials, several trees) is rejected with a message.
// nuka/nks.py is the same cooker in Python (offline use, procedural templates); tests compare the two array by array.
#include "nkb_scene.h"

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <set>

namespace nkb {
namespace {

constexpr int kInvalidArg = 1, kParseError = 5, kNotSupported = 7;
constexpr uint32_t kRevolute = 0, kPrismatic = 1, kFixed = 2, kFloating = 3;
constexpr uint32_t kSphere = 0, kCapsule = 1, kBox = 2, kPlane = 3, kCylinder = 7;
constexpr uint32_t kNoLink = 0xffffffffu;

// ---- a small JSON reader: objects keep their members in document order ----------------------------------------------------
struct Json {
    enum Kind { kNull, kBool, kNumber, kString, kArray, kObject } kind = kNull;
    bool boolean = false;
    double number = 0.0;
    std::string text;
    std::vector<Json> items;
    std::vector<std::pair<std::string, Json>> members;

    const Json* Find(const char* key) const {
        if (kind != kObject) return nullptr;
        for (const auto& m : members) if (m.first == key) return &m.second;
        return nullptr;
    }
    bool Has(const char* key) const { return Find(key) != nullptr; }
    double Number(const char* key, double fallback) const {
        const Json* v = Find(key);
        if (v == nullptr || v->kind == kNull) return fallback;
        if (v->kind == kBool) return v->boolean ? 1.0 : 0.0;
        if (v->kind != kNumber) throw Error(kParseError, std::string("scene field is not a number: ") + key);
        return v->number;
    }
    bool Truthy(const char* key) const {
        const Json* v = Find(key);
        if (v == nullptr) return false;
        switch (v->kind) {
            case kNull: return false;
            case kBool: return v->boolean;
            case kNumber: return v->number != 0.0;
            case kString: return !v->text.empty();
            case kArray: return !v->items.empty();
            default: return !v->members.empty();
        }
    }
    std::string String(const char* key, const std::string& fallback) const {
        const Json* v = Find(key);
        if (v == nullptr || v->kind != kString) return fallback;
        return v->text;
    }
};

class JsonReader {
   public:
    explicit JsonReader(const std::string& text) : s_(text) {}
    Json Document() {
        Json v = Value(0);
        Space();
        if (at_ != s_.size()) Fail("trailing characters after the document");
        return v;
    }

   private:
    [[noreturn]] void Fail(const char* what) const { throw Error(kParseError, std::string("scene JSON: ") + what + " at byte " + std::to_string(at_)); }
    void Space() { while (at_ < s_.size() && (s_[at_] == ' ' || s_[at_] == '\n' || s_[at_] == '\t' || s_[at_] == '\r')) ++at_; }
    bool Literal(const char* word) {
        const size_t n = std::strlen(word);
        if (s_.compare(at_, n, word) != 0) return false;
        at_ += n;
        return true;
    }
    std::string Text() {
        std::string out;
        ++at_;      // opening quote
        for (;;) {
            if (at_ >= s_.size()) Fail("unterminated string");
            const char c = s_[at_++];
            if (c == '"') return out;
            if (c != '\\') { out.push_back(c); continue; }
            if (at_ >= s_.size()) Fail("unterminated escape");
            const char e = s_[at_++];
            switch (e) {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'n': out.push_back('\n'); break;
                case 'r': out.push_back('\r'); break;
                case 't': out.push_back('\t'); break;
                case 'u': {
                    if (at_ + 4 > s_.size()) Fail("short \\u escape");
                    const unsigned long code = std::strtoul(s_.substr(at_, 4).c_str(), nullptr, 16);
                    at_ += 4;
                    // names only: keep the Basic Latin range, replace the rest
                    out.push_back(code < 0x80 ? static_cast<char>(code) : '?');
                    break;
                }
                default: Fail("unknown escape");
            }
        }
    }
    Json Value(int depth) {
        if (depth > 256) Fail("nesting too deep");
        Space();
        if (at_ >= s_.size()) Fail("unexpected end");
        Json v;
        const char c = s_[at_];
        if (c == '{') {
            v.kind = Json::kObject;
            ++at_;
            Space();
            if (at_ < s_.size() && s_[at_] == '}') { ++at_; return v; }
            for (;;) {
                Space();
                if (at_ >= s_.size() || s_[at_] != '"') Fail("object key expected");
                std::string key = Text();
                Space();
                if (at_ >= s_.size() || s_[at_] != ':') Fail("':' expected");
                ++at_;
                v.members.emplace_back(std::move(key), Value(depth + 1));
                Space();
                if (at_ < s_.size() && s_[at_] == ',') { ++at_; continue; }
                if (at_ < s_.size() && s_[at_] == '}') { ++at_; return v; }
                Fail("',' or '}' expected");
            }
        }
        if (c == '[') {
            v.kind = Json::kArray;
            ++at_;
            Space();
            if (at_ < s_.size() && s_[at_] == ']') { ++at_; return v; }
            for (;;) {
                v.items.push_back(Value(depth + 1));
                Space();
                if (at_ < s_.size() && s_[at_] == ',') { ++at_; continue; }
                if (at_ < s_.size() && s_[at_] == ']') { ++at_; return v; }
                Fail("',' or ']' expected");
            }
        }
        if (c == '"') { v.kind = Json::kString; v.text = Text(); return v; }
        if (Literal("true")) { v.kind = Json::kBool; v.boolean = true; return v; }
        if (Literal("false")) { v.kind = Json::kBool; return v; }
        if (Literal("null")) return v;
        if (Literal("NaN")) { v.kind = Json::kNumber; v.number = std::nan(""); return v; }
        if (Literal("Infinity")) { v.kind = Json::kNumber; v.number = INFINITY; return v; }
        if (Literal("-Infinity")) { v.kind = Json::kNumber; v.number = -INFINITY; return v; }
        const char* begin = s_.c_str() + at_;
        char* end = nullptr;
        const double number = std::strtod(begin, &end);
        if (end == begin) Fail("value expected");
        at_ += static_cast<size_t>(end - begin);
        v.kind = Json::kNumber;
        v.number = number;
        return v;
    }
    const std::string& s_;
    size_t at_ = 0;
};

// ---- small double-precision algebra (the cooker computes in double and stores float, as the Python cooker does) -------------
struct D3 { double x = 0, y = 0, z = 0; };
struct D4 { double w = 1, x = 0, y = 0, z = 0; };
struct M3 { double m[3][3] = {{0, 0, 0}, {0, 0, 0}, {0, 0, 0}}; };

M3 QuatToMatrix(D4 q) {
    const double w = q.w, x = q.x, y = q.y, z = q.z;
    M3 r;
    r.m[0][0] = 1 - 2 * (y * y + z * z); r.m[0][1] = 2 * (x * y - w * z); r.m[0][2] = 2 * (x * z + w * y);
    r.m[1][0] = 2 * (x * y + w * z); r.m[1][1] = 1 - 2 * (x * x + z * z); r.m[1][2] = 2 * (y * z - w * x);
    r.m[2][0] = 2 * (x * z - w * y); r.m[2][1] = 2 * (y * z + w * x); r.m[2][2] = 1 - 2 * (x * x + y * y);
    return r;
}
D4 QuatMul(D4 a, D4 b) {
    return {a.w * b.w - a.x * b.x - a.y * b.y - a.z * b.z, a.w * b.x + a.x * b.w + a.y * b.z - a.z * b.y,
            a.w * b.y - a.x * b.z + a.y * b.w + a.z * b.x, a.w * b.z + a.x * b.y - a.y * b.x + a.z * b.w};
}
D3 Apply(const M3& r, D3 v) {
    return {r.m[0][0] * v.x + r.m[0][1] * v.y + r.m[0][2] * v.z, r.m[1][0] * v.x + r.m[1][1] * v.y + r.m[1][2] * v.z,
            r.m[2][0] * v.x + r.m[2][1] * v.y + r.m[2][2] * v.z};
}

struct Frame { D3 pos; D4 quat; };
Frame FrameOf(const Json& record, const char* key) {
    Frame f;
    const Json* frame = record.Find(key);
    if (frame == nullptr || frame->kind != Json::kObject) return f;
    if (const Json* p = frame->Find("pos")) {
        if (p->kind != Json::kArray || p->items.size() != 3) throw Error(kParseError, "scene frame: pos needs three numbers");
        f.pos = {p->items[0].number, p->items[1].number, p->items[2].number};
    }
    if (const Json* q = frame->Find("quat")) {
        if (q->kind != Json::kArray || q->items.size() != 4) throw Error(kParseError, "scene frame: quat needs four numbers");
        f.quat = {q->items[0].number, q->items[1].number, q->items[2].number, q->items[3].number};
    }
    return f;
}
bool IsIdentity(D4 q) { return std::fabs(std::fabs(q.w) - 1.0) <= 1e-9; }
bool IsZero(D3 v) { return std::fmax(std::fabs(v.x), std::fmax(std::fabs(v.y), std::fabs(v.z))) == 0.0; }

// ---- the template under construction (rows as the cooked template stores them) ------------------------------------------------
struct Shape { uint32_t kind = kSphere; double params[4] = {0, 0, 0, 0}; };

Shape ShapeOf(const Json& cs) {
    const std::string kind = cs.String("type", "");
    Shape s;
    if (kind == "sphere") { s.kind = kSphere; s.params[0] = cs.Number("radius", 0.0); return s; }
    if (kind == "capsule") { s.kind = kCapsule; s.params[0] = cs.Number("radius", 0.0); s.params[1] = cs.Number("half_height", 0.0); return s; }
    if (kind == "cylinder") { s.kind = kCylinder; s.params[0] = cs.Number("radius", 0.0); s.params[1] = cs.Number("half_height", 0.0); return s; }
    if (kind == "box") {
        const Json* he = cs.Find("half_extents");
        if (he == nullptr || he->kind != Json::kArray || he->items.size() != 3) throw Error(kParseError, "box shape without half_extents");
        s.kind = kBox;
        for (int k = 0; k < 3; ++k) s.params[k] = he->items[k].number;
        return s;
    }
    throw Error(kNotSupported, "collision shape type '" + kind + "' has no analytic manifold here");
}

struct LinkRow {
    uint32_t parent = kNoLink, jtype = kFixed, body = 0, geom = 0;
    D3 axis{0, 0, 1}, offset, com, local_pos, geom_pos;
    D4 local_quat, geom_quat;
    double mass = 0, q0 = 0, kp = 0, kd = 0, force_limit = 0, damping = 0, armature = 0, frictionloss = 0;
    bool limited = false;
    double lower = 0, upper = 0;
    float inertia[36] = {0};
    std::string name;          // the joint whose child the body is, else the body's own (src/c_abi/world.cpp:1186-1199)
};
struct BodyRow {
    uint32_t kind = kSphere, contype = 0, conaffinity = 0, group = 0, link = kNoLink, geom = 0;
    int32_t body_id = 0;
    double params[4] = {0, 0, 0, 0}, mu = 1, inv_mass = 0, inv_inertia[3] = {0, 0, 0};
    D3 inertial_pos, geom_pos;
    D4 inertial_quat, geom_quat;
    double pose[7] = {0, 0, 0, 1, 0, 0, 0};
};

// [[Icom + m (c.c 1 - c c^T), m c^x], [-m c^x, m 1]] about the link frame, angular first
// (runtime/articulation/articulation_state.cpp:307-342).
void SpatialInertia(double mass, const M3& about_com, D3 c, float out[36]) {
    double I[6][6] = {{0}};
    if (mass > 0.0) {
        const double cc = c.x * c.x + c.y * c.y + c.z * c.z;
        const double v[3] = {c.x, c.y, c.z};
        for (int i = 0; i < 3; ++i)
            for (int j = 0; j < 3; ++j) I[i][j] = about_com.m[i][j] + mass * ((i == j ? cc : 0.0) - v[i] * v[j]);
        const double cx[3][3] = {{0, -c.z, c.y}, {c.z, 0, -c.x}, {-c.y, c.x, 0}};
        for (int i = 0; i < 3; ++i)
            for (int j = 0; j < 3; ++j) { I[i][3 + j] = mass * cx[i][j]; I[3 + i][j] = -mass * cx[i][j]; }
        for (int i = 0; i < 3; ++i) I[3 + i][3 + i] = mass;
    }
    for (int i = 0; i < 6; ++i)
        for (int j = 0; j < 6; ++j) out[i * 6 + j] = static_cast<float>(I[i][j]);
}

class Builder {
   public:
    std::vector<LinkRow> links;
    std::vector<BodyRow> bodies;
    std::set<uint64_t> excluded;
    bool extra_shapes = false;
    double base_pose[7] = {0, 0, 0, 1, 0, 0, 0};

    uint32_t AddLink(const LinkRow& row, const Shape* shape, double mu, uint32_t contype, uint32_t conaffinity) {
        const uint32_t index = static_cast<uint32_t>(links.size()), body = static_cast<uint32_t>(bodies.size());
        LinkRow l = row;
        l.body = body;
        l.geom = shape != nullptr ? 1u : 0u;
        links.push_back(l);
        BodyRow b;
        if (shape != nullptr) { b.kind = shape->kind; std::memcpy(b.params, shape->params, sizeof(b.params)); b.contype = contype; b.conaffinity = conaffinity; }
        b.body_id = static_cast<int32_t>(body);
        b.link = index;
        b.mu = mu;
        b.geom = l.geom; b.geom_pos = l.geom_pos; b.geom_quat = l.geom_quat;
        bodies.push_back(b);
        if (l.parent != kNoLink) {
            const uint64_t a = links[l.parent].body, c = body;
            excluded.insert((std::min(a, c) << 32) | std::max(a, c));
        }
        return index;
    }
    void AddLinkShape(uint32_t link, const Shape& shape, const Frame& local, double mu, uint32_t contype, uint32_t conaffinity) {
        BodyRow b;
        b.kind = shape.kind; std::memcpy(b.params, shape.params, sizeof(b.params));
        b.contype = contype; b.conaffinity = conaffinity;
        b.body_id = static_cast<int32_t>(bodies.size());
        b.link = link; b.mu = mu; b.geom = 1u; b.geom_pos = local.pos; b.geom_quat = local.quat;
        bodies.push_back(b);
        extra_shapes = true;
    }
    void AddFreeBody(const Shape& shape, double mass, const double inertia[3], const Frame& pose, double mu, uint32_t contype, uint32_t conaffinity) {
        BodyRow b;
        b.kind = shape.kind; std::memcpy(b.params, shape.params, sizeof(b.params));
        b.contype = contype; b.conaffinity = conaffinity;
        b.body_id = static_cast<int32_t>(bodies.size());
        b.mu = mu; b.inv_mass = 1.0 / mass;
        for (int k = 0; k < 3; ++k) b.inv_inertia[k] = 1.0 / inertia[k];
        const double p[7] = {pose.pos.x, pose.pos.y, pose.pos.z, pose.quat.w, pose.quat.x, pose.quat.y, pose.quat.z};
        std::memcpy(b.pose, p, sizeof(p));
        bodies.push_back(b);
    }
    void AddPlane(double height, double mu, uint32_t contype, uint32_t conaffinity) {
        BodyRow b;
        b.kind = kPlane; b.contype = contype; b.conaffinity = conaffinity; b.body_id = -1; b.mu = mu;
        b.pose[2] = height;
        bodies.push_back(b);
    }
};

// ---- the container writer ---------------------------------------------------------------------------------------------------------
class Blob {
   public:
    Blob() { bytes_.assign({'N', 'K', 'T', '1', 0, 0, 0, 0}); }
    template <typename T>
    void Add(const char* name, uint32_t dtype, const std::vector<T>& values) {
        char field[32] = {0};
        std::strncpy(field, name, 31);
        Append(field, 32);
        const uint32_t head[2] = {dtype, 0u};
        Append(head, 8);
        const uint64_t n = values.size();
        Append(&n, 8);
        const size_t raw = values.size() * sizeof(T);
        if (raw != 0) Append(values.data(), raw);
        const char zeros[8] = {0};
        Append(zeros, (8 - raw % 8) % 8);
        ++count_;
    }
    void F32(const char* name, const std::vector<float>& v) { Add(name, 0u, v); }
    void U32(const char* name, const std::vector<uint32_t>& v) { Add(name, 1u, v); }
    void I32(const char* name, const std::vector<int32_t>& v) { Add(name, 2u, v); }
    void U64(const char* name, const std::vector<uint64_t>& v) { Add(name, 3u, v); }
    std::vector<uint8_t> Finish() {
        std::memcpy(bytes_.data() + 4, &count_, 4);
        return bytes_;
    }

   private:
    void Append(const void* p, size_t n) {
        const uint8_t* b = static_cast<const uint8_t*>(p);
        bytes_.insert(bytes_.end(), b, b + n);
    }
    std::vector<uint8_t> bytes_;
    uint32_t count_ = 0;
};

uint32_t Bits(const Json& shape, const char* key) { return static_cast<uint32_t>(static_cast<long long>(shape.Number(key, 1.0))); }

bool IsGround(const Json& node) {
    const Json* rb = node.Find("rigid_body");
    if (rb == nullptr || !rb->Truthy("is_static")) return false;
    const Json* children = node.Find("children");
    if (children == nullptr || children->kind != Json::kArray) return false;
    bool plane = false;
    for (const Json& c : children->items) {
        if (c.Has("rigid_body")) return false;
        if (const Json* cs = c.Find("collision_shape")) plane |= cs->String("type", "") == "plane";
    }
    return plane;
}
bool HasChildBodies(const Json& node) {
    const Json* children = node.Find("children");
    if (children == nullptr || children->kind != Json::kArray) return false;
    for (const Json& c : children->items) if (c.Has("rigid_body")) return true;
    return false;
}
std::vector<const Json*> ShapesOf(const Json& node) {
    std::vector<const Json*> shapes;
    if (const Json* children = node.Find("children"))
        if (children->kind == Json::kArray)
            for (const Json& c : children->items)
                if (const Json* cs = c.Find("collision_shape")) shapes.push_back(cs);
    return shapes;
}

class Cooker {
   public:
    Cooker(const CookOptions& o) : o_(o), self_collision_(o.self_collision || o.scene_filters) {}

    std::vector<uint8_t> Cook(const Json& scene) {
        if (scene.kind != Json::kObject || scene.Number("nks_version", 0.0) != 1.0) throw Error(kNotSupported, "unsupported nks_version");
        std::vector<const Json*> grounds, roots, free_bodies;
        if (const Json* tree = scene.Find("tree"))
            if (tree->kind == Json::kArray)
                for (const Json& n : tree->items) {
                    const Json* rb = n.Find("rigid_body");
                    if (rb == nullptr) continue;
                    if (IsGround(n)) grounds.push_back(&n);
                    else if (HasChildBodies(n) || rb->Truthy("is_static")) roots.push_back(&n);
                    else free_bodies.push_back(&n);
                }
        if (roots.size() > 1) throw Error(kNotSupported, "at most one articulated tree is supported");
        if (!roots.empty()) { AddBody(*roots[0], kNoLink); ExcludeWelded(); }
        for (const Json* node : free_bodies) AddFree(*node);      // in document order, after the articulation's rows
        for (const Json* g : grounds) {
            const Json* plane = nullptr;
            for (const Json* cs : ShapesOf(*g)) if (cs->String("type", "") == "plane") { plane = cs; break; }
            const Frame pose = FrameOf(*g, "transform");
            if (!IsIdentity(pose.quat) || !IsZero(FrameOf(*plane, "local").pos))
                throw Error(kNotSupported, "only horizontal ground planes at the body origin are carried over");
            const uint32_t contype = o_.scene_filters ? Bits(*plane, "contype") : 2u, conaffinity = o_.scene_filters ? Bits(*plane, "conaffinity") : 1u;
            tb_.AddPlane(pose.pos.z, plane->Number("friction_mu", 1.0), contype, conaffinity);
        }
        if (grounds.empty() && o_.default_ground) tb_.AddPlane(o_.ground_height, o_.ground_mu, 2u, 1u);
        return Pack();
    }

   private:
    void AddBody(const Json& node, uint32_t parent_link) {
        const Json& rb = *node.Find("rigid_body");
        const Frame pose = FrameOf(node, "transform");
        const Json* joint = node.Find("joint");
        static const Json none;
        LinkRow l;
        l.parent = parent_link;
        l.name = joint != nullptr ? joint->String("name", "") : std::string();
        if (l.name.empty()) l.name = node.String("name", "");
        if (parent_link == kNoLink) {
            l.jtype = rb.Truthy("is_static") ? kFixed : kFloating;
            const double bp[7] = {pose.pos.x, pose.pos.y, pose.pos.z, pose.quat.w, pose.quat.x, pose.quat.y, pose.quat.z};
            std::memcpy(tb_.base_pose, bp, sizeof(bp));
            if (l.jtype == kFixed) { l.local_pos = pose.pos; l.local_quat = pose.quat; }
            joint = &none;
        } else {
            std::string type = "fixed";
            if (joint != nullptr && joint->kind == Json::kObject) type = joint->String("type", "");
            else joint = &none;
            if (type == "revolute" || type == "hinge") l.jtype = kRevolute;
            else if (type == "prismatic" || type == "slide") l.jtype = kPrismatic;
            else if (type == "fixed") l.jtype = kFixed;
            else throw Error(kNotSupported, "joint type '" + type + "' is not supported");
            const Frame pf = FrameOf(*joint, "parent_frame"), cf = FrameOf(*joint, "child_frame");
            if (!IsZero(cf.pos) || !IsIdentity(cf.quat)) throw Error(kNotSupported, "joints with a non-identity child frame are not supported");
            l.local_pos = Apply(QuatToMatrix(pf.quat), pose.pos);
            l.local_quat = QuatMul(pf.quat, pose.quat);
            l.offset = pf.pos;
            if (const Json* axis = joint->Find("axis")) {
                if (axis->kind != Json::kArray || axis->items.size() != 3) throw Error(kParseError, "joint axis needs three numbers");
                // as the reference cooks it (src/scene/cooker.cpp:680, math::Vec3::Normalized): float components over the
                // float length, zero when shorter than 1e-12
                const float x = (float)axis->items[0].number, y = (float)axis->items[1].number, z = (float)axis->items[2].number;
                const volatile float xx = x * x, yy = y * y, zz = z * z;      // each product rounded on its own, no contraction
                const volatile float sum = xx + yy;
                const float length = std::sqrt((float)(sum + zz));
                if (length < 1e-12f) l.axis = {0.0, 0.0, 0.0};
                else l.axis = {(double)(x / length), (double)(y / length), (double)(z / length)};
            }
        }
        const Frame inertial = FrameOf(rb, "inertial");
        double diag[3] = {0, 0, 0};
        if (const Json* in = rb.Find("inertia")) {
            if (in->kind != Json::kArray || in->items.size() != 3) throw Error(kParseError, "rigid_body inertia needs three numbers");
            for (int k = 0; k < 3; ++k) diag[k] = in->items[k].number;
        }
        // R diag R^T, in the product order of the Python cooker: (R diag) R^T
        const M3 R = QuatToMatrix(inertial.quat);
        M3 about_com;
        for (int i = 0; i < 3; ++i)
            for (int j = 0; j < 3; ++j) {
                double sum = 0.0;
                for (int k = 0; k < 3; ++k) sum += (R.m[i][k] * diag[k]) * R.m[j][k];
                about_com.m[i][j] = sum;
            }
        const bool static_root = parent_link == kNoLink && l.jtype == kFixed;     // a static body carries no inertia
        l.mass = static_root ? 0.0 : rb.Number("mass", 0.0);
        l.com = inertial.pos;
        SpatialInertia(l.mass, about_com, l.com, l.inertia);
        const std::vector<const Json*> shapes = ShapesOf(node);
        const Json* first = shapes.empty() ? nullptr : shapes[0];
        const bool single = l.jtype == kRevolute || l.jtype == kPrismatic;
        if (single) {
            l.lower = joint->Number("lower_limit", 0.0); l.upper = joint->Number("upper_limit", 0.0);
            l.limited = l.lower < l.upper;
            l.q0 = joint->Number("initial_position", 0.0);
            l.frictionloss = joint->Number("frictionloss", 0.0);
            l.damping = joint->Number("damping", 0.0);
            l.armature = joint->Number("armature", 0.0);
            if (joint->Number("stiffness", 0.0) != 0.0) throw Error(kNotSupported, "joint springs are not carried over");
            const Json* act = node.Find("actuator");
            if (act != nullptr && act->kind == Json::kObject) {
                if (act->String("type", "") != "position") throw Error(kNotSupported, "only position actuators are carried over");
                // a position actuator's gain is the drive stiffness; without an authored damping the reference uses the
                // critically damped 2 sqrt(gain) (scene_ir.hpp:335-336)
                const double gain = act->Number("gain", 0.0);
                l.kp = gain;
                l.kd = act->Has("damping") ? act->Number("damping", 0.0) : 2.0 * std::sqrt(gain);
                l.force_limit = act->Number("force_limit", 0.0);
            } else { l.kp = o_.kp; l.kd = o_.kd; }
        }
        uint32_t contype = 1u, conaffinity = 0u;
        Shape shape;
        double mu = 1.0;
        if (first != nullptr) {
            shape = ShapeOf(*first);
            const Frame local = FrameOf(*first, "local");
            l.geom_pos = local.pos; l.geom_quat = local.quat;
            mu = first->Number("friction_mu", 1.0);
            if (self_collision_) { contype = Bits(*first, "contype"); conaffinity = Bits(*first, "conaffinity"); }
        }
        const uint32_t link = tb_.AddLink(l, first != nullptr ? &shape : nullptr, mu, contype, conaffinity);
        if (first != nullptr) ++shape_rows_;
        for (size_t k = 1; k < shapes.size(); ++k) {
            const Json& cs = *shapes[k];
            const uint32_t ct = self_collision_ ? Bits(cs, "contype") : 1u, ca = self_collision_ ? Bits(cs, "conaffinity") : 0u;
            tb_.AddLinkShape(link, ShapeOf(cs), FrameOf(cs, "local"), cs.Number("friction_mu", 1.0), ct, ca);
            ++shape_rows_;
        }
        if (const Json* children = node.Find("children"))
            if (children->kind == Json::kArray)
                for (const Json& c : children->items)
                    if (c.Has("rigid_body")) AddBody(c, link);
    }

    // The reference's weld rule (src/scene/cooker.cpp:505-536, MuJoCo's weldbody and filterparent): links joined by fixed
    // joints form a cluster; no pair inside a cluster, and none between a cluster and the cluster of its parent link.
    // Without fixed joints this is the parent-child exclusion AddLink already applies.
    void ExcludeWelded() {
        const uint32_t L = static_cast<uint32_t>(tb_.links.size());
        auto weld = [&](uint32_t l) {
            while (tb_.links[l].parent != kNoLink && tb_.links[l].jtype == kFixed) l = tb_.links[l].parent;
            return l;
        };
        std::vector<std::vector<uint32_t>> clusters(L), rows(L);
        for (uint32_t l = 0; l < L; ++l) clusters[weld(l)].push_back(l);
        for (uint32_t row = 0; row < tb_.bodies.size(); ++row)
            if (tb_.bodies[row].link != kNoLink) rows[tb_.bodies[row].link].push_back(row);
        auto exclude = [&](uint32_t a, uint32_t b) {
            if (a == b) return;
            for (uint64_t ra : rows[a])
                for (uint64_t rb : rows[b]) tb_.excluded.insert((std::min(ra, rb) << 32) | std::max(ra, rb));
        };
        for (uint32_t root = 0; root < L; ++root) {
            const std::vector<uint32_t>& members = clusters[root];
            for (size_t i = 0; i < members.size(); ++i)
                for (size_t k = i + 1; k < members.size(); ++k) exclude(members[i], members[k]);
            if (members.empty() || tb_.links[root].parent == kNoLink) continue;
            for (uint32_t other : clusters[weld(tb_.links[root].parent)])
                for (uint32_t member : members) exclude(member, other);
        }
    }

    void AddFree(const Json& node) {
        const Json& rb = *node.Find("rigid_body");
        const std::vector<const Json*> shapes = ShapesOf(node);
        if (shapes.size() != 1) throw Error(kNotSupported, "a free body needs exactly one collision shape");
        const Json& cs = *shapes[0];
        const Frame pose = FrameOf(node, "transform"), inertial = FrameOf(rb, "inertial");
        if (!IsZero(FrameOf(cs, "local").pos) || !IsZero(inertial.pos) || !IsIdentity(inertial.quat))
            throw Error(kNotSupported, "free bodies with an offset shape or inertial frame are not carried over");
        const Json* in = rb.Find("inertia");
        if (in == nullptr || in->kind != Json::kArray || in->items.size() != 3 || !rb.Has("mass")) throw Error(kParseError, "free body without mass or inertia");
        const double inertia[3] = {in->items[0].number, in->items[1].number, in->items[2].number};
        tb_.AddFreeBody(ShapeOf(cs), rb.Number("mass", 0.0), inertia, pose, cs.Number("friction_mu", 1.0), Bits(cs, "contype"), Bits(cs, "conaffinity"));
        ++shape_rows_;
    }

    std::vector<uint8_t> Pack() {
        const uint32_t L = static_cast<uint32_t>(tb_.links.size()), B = static_cast<uint32_t>(tb_.bodies.size());
        uint32_t max_contacts = o_.max_contacts;
        if (max_contacts == 0u) max_contacts = std::max(shape_rows_, 1u);
        else if (max_contacts == kEveryAdmissiblePair) max_contacts = 1u;      // a placeholder: the caller counts the admissible pairs and cooks again
        Blob out;
        out.F32("cfg_f", {o_.dt, 0.0f, 0.0f, -9.81f, 0.3f, 0.001f, 0.0f, 3.0e38f, 0.0f, 1.0e-5f});
        out.U32("cfg_u", {o_.vel_iters, o_.pos_iters, max_contacts, 0u, L, B});
        std::vector<uint32_t> parent, jtype, link_body, geom_kind, limit_flags;
        std::vector<float> axis, local_pos, local_quat, offset, com, inertia, damping, armature, frictionloss, lower, upper, geom_pos, geom_quat, q0, kp, kd, force_limit;
        auto push3 = [](std::vector<float>& v, D3 a) { v.push_back((float)a.x); v.push_back((float)a.y); v.push_back((float)a.z); };
        auto push4 = [](std::vector<float>& v, D4 a) { v.push_back((float)a.w); v.push_back((float)a.x); v.push_back((float)a.y); v.push_back((float)a.z); };
        for (const LinkRow& l : tb_.links) {
            parent.push_back(l.parent); jtype.push_back(l.jtype); link_body.push_back(l.body); geom_kind.push_back(l.geom);
            limit_flags.push_back(l.limited ? 3u : 0u);
            push3(axis, l.axis); push3(local_pos, l.local_pos); push4(local_quat, l.local_quat); push3(offset, l.offset); push3(com, l.com);
            inertia.insert(inertia.end(), l.inertia, l.inertia + 36);
            damping.push_back((float)l.damping); armature.push_back((float)l.armature); frictionloss.push_back((float)l.frictionloss);
            lower.push_back(l.limited ? (float)l.lower : 0.0f); upper.push_back(l.limited ? (float)l.upper : 0.0f);
            push3(geom_pos, l.geom_pos); push4(geom_quat, l.geom_quat);
            q0.push_back((float)l.q0); kp.push_back((float)l.kp); kd.push_back((float)l.kd); force_limit.push_back((float)l.force_limit);
        }
        out.U32("parent", parent); out.U32("jtype", jtype); out.U32("link_body", link_body); out.U32("geom_kind", geom_kind);
        out.U32("limit_flags", limit_flags);
        out.F32("axis", axis); out.F32("local_pos", local_pos); out.F32("local_quat", local_quat); out.F32("parent_offset", offset); out.F32("com", com);
        out.F32("inertia", inertia); out.F32("damping", damping); out.F32("armature", armature); out.F32("frictionloss", frictionloss);
        out.F32("stiffness", std::vector<float>(L, 0.0f)); out.F32("spring_ref", std::vector<float>(L, 0.0f));
        out.F32("limit_lower", lower); out.F32("limit_upper", upper); out.F32("geom_pos", geom_pos); out.F32("geom_quat", geom_quat);
        out.F32("q0", q0);
        std::vector<float> base(7);
        for (int k = 0; k < 7; ++k) base[k] = (float)tb_.base_pose[k];
        out.F32("base_pose0", base);
        out.F32("kp0", kp); out.F32("kd0", kd); out.F32("force_limit0", force_limit);
        std::vector<uint32_t> shape_kind, contype, conaffinity, group, body_to_link, body_geom_kind;
        std::vector<int32_t> body_id;
        std::vector<float> params, mu, inv_mass, inv_inertia, inertial_pos, inertial_quat, body_pose, body_geom_pos, body_geom_quat;
        for (const BodyRow& b : tb_.bodies) {
            shape_kind.push_back(b.kind); contype.push_back(b.contype); conaffinity.push_back(b.conaffinity); group.push_back(b.group);
            body_to_link.push_back(b.link); body_id.push_back(b.body_id);
            for (int k = 0; k < 4; ++k) params.push_back((float)b.params[k]);
            mu.push_back((float)b.mu); inv_mass.push_back((float)b.inv_mass);
            for (int k = 0; k < 3; ++k) inv_inertia.push_back((float)b.inv_inertia[k]);
            push3(inertial_pos, b.inertial_pos); push4(inertial_quat, b.inertial_quat);
            for (int k = 0; k < 7; ++k) body_pose.push_back((float)b.pose[k]);
            body_geom_kind.push_back(b.geom); push3(body_geom_pos, b.geom_pos); push4(body_geom_quat, b.geom_quat);
        }
        out.U32("shape_kind", shape_kind); out.U32("contype", contype); out.U32("conaffinity", conaffinity); out.U32("group", group);
        out.U32("body_to_link", body_to_link); out.I32("body_id", body_id);
        out.F32("shape_params", params); out.F32("mu", mu); out.F32("inv_mass", inv_mass); out.F32("inv_inertia", inv_inertia);
        out.F32("inertial_pos", inertial_pos); out.F32("inertial_quat", inertial_quat); out.F32("body_pose0", body_pose);
        std::set<uint64_t> excluded = tb_.excluded;
        if (tb_.extra_shapes) {
            // several rows per link: per-row shape frames, and no pairs inside a link or between a link and its parent
            out.U32("body_geom_kind", body_geom_kind); out.F32("body_geom_pos", body_geom_pos); out.F32("body_geom_quat", body_geom_quat);
            for (uint64_t a = 0; a < B; ++a) {
                const uint32_t la = tb_.bodies[a].link;
                if (la == kNoLink) continue;
                for (uint64_t b = a + 1; b < B; ++b) {
                    const uint32_t lb = tb_.bodies[b].link;
                    if (lb == kNoLink) continue;
                    if (la == lb || tb_.links[la].parent == lb || tb_.links[lb].parent == la) excluded.insert((a << 32) | b);
                }
            }
        }
        out.U64("excluded", std::vector<uint64_t>(excluded.begin(), excluded.end()));
        if (o_.max_points != 0u) out.U32("max_points", {o_.max_points});
        bool named = false;
        for (const LinkRow& l : tb_.links) named |= !l.name.empty();
        if (named) {        // NUL-terminated names in link order, padded to whole words
            std::string raw;
            for (const LinkRow& l : tb_.links) { raw += l.name; raw.push_back('\0'); }
            while (raw.size() % 4u != 0u) raw.push_back('\0');
            std::vector<uint32_t> words(raw.size() / 4u);
            std::memcpy(words.data(), raw.data(), raw.size());
            out.U32("link_names", words);
        }
        return out.Finish();
    }

    CookOptions o_;
    bool self_collision_;
    Builder tb_;
    uint32_t shape_rows_ = 0;
};

}  // namespace

std::vector<uint8_t> CookScene(const std::string& json_text, const CookOptions& options) {
    if (!(options.dt > 0.0f) || !std::isfinite(options.dt)) throw Error(kInvalidArg, "cook options: dt must be positive");
    JsonReader reader(json_text);
    const Json scene = reader.Document();
    Cooker cooker(options);
    return cooker.Cook(scene);
}

std::vector<uint8_t> CookSceneForWorld(const std::string& json_text, const CookOptions& options) {
    std::vector<uint8_t> blob = CookScene(json_text, options);
    if (options.max_contacts != kEveryAdmissiblePair) return blob;
    // one candidate slot per pair the filters admit, the reference's budget: count them with the template parser's own rule
    const HostTemplate parsed = HostTemplate::Parse(blob.data(), blob.size());
    const bool none = parsed.adm_pairs.size() == 1 && parsed.adm_pairs[0] == 0u;
    CookOptions narrowed = options;
    narrowed.max_contacts = none ? 1u : static_cast<uint32_t>(parsed.adm_pairs.size());
    return CookScene(json_text, narrowed);
}

bool LooksLikeScene(const std::string& bytes) {
    for (char c : bytes) {
        if (c == ' ' || c == '\n' || c == '\t' || c == '\r') continue;
        return c == '{';
    }
    return false;
}

}  // namespace nkb
