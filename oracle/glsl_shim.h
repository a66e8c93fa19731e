// Test infrastructure only. Nothing in the product path includes this file.
//
// A small set of GLSL ES 3.00 types and built-ins, written as plain C++, so
// that the reference runtime's fragment shaders (ogl_runtime/opengl/nn/glsl/*.glsl)
// compile UNMODIFIED as C++ translation units. A "texture" is a linear float
// array of RGBA32F texels with a row width; texelFetch indexes it. The build
// recipe (oracle/Makefile) includes each shader inside its own namespace and
// drives main() once per output texel, which is what the reference's
// two-triangle draw does (ogl_runtime/opengl/core/program.cc:113-130).
#ifndef ORACLE_GLSL_SHIM_H_
#define ORACLE_GLSL_SHIM_H_
#include <cmath>
#include <algorithm>

namespace glsl {

struct vec2 { float x, y; };

struct ivec2 {
    int x, y;
    ivec2() : x(0), y(0) {}
    ivec2(int a, int b) : x(a), y(b) {}
    // float -> int conversion truncates toward zero, as in GLSL
    explicit ivec2(const vec2& v) : x(int(v.x)), y(int(v.y)) {}
};
struct ivec3 { int x, y, z; };
struct ivec4 {
    int x, y, z, w;
    int operator[](int i) const { return (&x)[i]; }
};

struct vec4 {
    float x, y, z, w;
    vec4() : x(0), y(0), z(0), w(0) {}
    explicit vec4(float s) : x(s), y(s), z(s), w(s) {}
    explicit vec4(double s) : x(float(s)), y(float(s)), z(float(s)), w(float(s)) {}
    vec4(float a, float b, float c, float d) : x(a), y(b), z(c), w(d) {}
    vec4& operator+=(const vec4& o) { x += o.x; y += o.y; z += o.z; w += o.w; return *this; }
};
inline vec4 operator+(const vec4& a, const vec4& b) { return vec4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
inline vec4 operator-(const vec4& a, const vec4& b) { return vec4(a.x - b.x, a.y - b.y, a.z - b.z, a.w - b.w); }
inline vec4 operator*(const vec4& a, const vec4& b) { return vec4(a.x * b.x, a.y * b.y, a.z * b.z, a.w * b.w); }
inline vec4 operator/(const vec4& a, const vec4& b) { return vec4(a.x / b.x, a.y / b.y, a.z / b.z, a.w / b.w); }
inline vec4 operator*(float s, const vec4& a) { return vec4(s * a.x, s * a.y, s * a.z, s * a.w); }
inline vec4 operator*(const vec4& a, float s) { return vec4(a.x * s, a.y * s, a.z * s, a.w * s); }
inline vec4 operator/(const vec4& a, float s) { return vec4(a.x / s, a.y / s, a.z / s, a.w / s); }
inline vec4 operator+(const vec4& a, float s) { return vec4(a.x + s, a.y + s, a.z + s, a.w + s); }

inline vec4 max(const vec4& a, const vec4& b) { return vec4(std::max(a.x, b.x), std::max(a.y, b.y), std::max(a.z, b.z), std::max(a.w, b.w)); }
inline vec4 min(const vec4& a, const vec4& b) { return vec4(std::min(a.x, b.x), std::min(a.y, b.y), std::min(a.z, b.z), std::min(a.w, b.w)); }
// GLSL clamp(x, lo, hi) is min(max(x, lo), hi)
inline vec4 clamp(const vec4& v, const vec4& lo, const vec4& hi) { return min(max(v, lo), hi); }
inline vec4 sqrt(const vec4& a) { return vec4(std::sqrt(a.x), std::sqrt(a.y), std::sqrt(a.z), std::sqrt(a.w)); }
inline vec4 exp(const vec4& a) { return vec4(std::exp(a.x), std::exp(a.y), std::exp(a.z), std::exp(a.w)); }
using std::sqrt;
using std::exp;
using std::max;
using std::min;

// Column-major 4x4: mat4(c0,c1,c2,c3) * v = c0*v.x + c1*v.y + c2*v.z + c3*v.w,
// summed left to right.
struct mat4 {
    vec4 c0, c1, c2, c3;
    mat4(const vec4& a, const vec4& b, const vec4& c, const vec4& d) : c0(a), c1(b), c2(c), c3(d) {}
};
inline vec4 operator*(const mat4& m, const vec4& v) {
    return ((m.c0 * v.x + m.c1 * v.y) + m.c2 * v.z) + m.c3 * v.w;
}

// A texture: RGBA32F texels, `width` texels per row, row-major.
struct sampler2D {
    const float* data;
    int width;
    int height;
};
inline vec4 texelFetch(const sampler2D& s, const ivec2& p, int /*lod*/) {
    const float* t = s.data + (size_t(p.y) * size_t(s.width) + size_t(p.x)) * 4;
    return vec4(t[0], t[1], t[2], t[3]);
}
inline ivec2 textureSize(const sampler2D& s, int /*lod*/) { return ivec2(s.width, s.height); }

struct FragCoord { vec2 xy; };

}  // namespace glsl

#endif  // ORACLE_GLSL_SHIM_H_
