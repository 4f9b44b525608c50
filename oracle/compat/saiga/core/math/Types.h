// Stand-in for the one saiga header that the reference's rendering/PointBlending.h includes (the saiga library is an
// empty submodule in the reference tree).  It supplies just the vector / matrix vocabulary that header uses, written
// from scratch: fixed-size column vectors with (), [], x(), y(), array().floor(), setZero(), and a dense Matrix.
// TEST INFRASTRUCTURE ONLY: used to compile the reference's blend algebra into oracle/_ref/libref_blend.so.
#pragma once
#include <cassert>
#include <cmath>

#define HD
#define SAIGA_ASSERT(x) assert(x)

namespace Saiga
{
template <typename T, int R, int C>
struct Matrix
{
    T m[R * C];
    Matrix() { setZero(); }
    void setZero()
    {
        for (int i = 0; i < R * C; ++i) m[i] = T(0);
    }
    T& operator()(int r, int c) { return m[r * C + c]; }
    const T& operator()(int r, int c) const { return m[r * C + c]; }
    // column-vector accessors (C == 1)
    T& operator()(int i) { return m[i]; }
    const T& operator()(int i) const { return m[i]; }
    T& operator[](int i) { return m[i]; }
    const T& operator[](int i) const { return m[i]; }
    T& x() { return m[0]; }
    T& y() { return m[1]; }
    const T& x() const { return m[0]; }
    const T& y() const { return m[1]; }
    struct ArrayProxy
    {
        const Matrix& v;
        Matrix floor() const
        {
            Matrix r;
            for (int i = 0; i < R * C; ++i) r.m[i] = std::floor(v.m[i]);
            return r;
        }
    };
    ArrayProxy array() const { return ArrayProxy{*this}; }
    Matrix operator-(const Matrix& o) const
    {
        Matrix r;
        for (int i = 0; i < R * C; ++i) r.m[i] = m[i] - o.m[i];
        return r;
    }
};
using vec2 = Matrix<float, 2, 1>;
using vec4 = Matrix<float, 4, 1>;
}  // namespace Saiga
