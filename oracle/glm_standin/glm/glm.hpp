// Stand-in for the subset of the GLM maths library that the reference's gsplat operators use.
//
// TEST INFRASTRUCTURE. The reference's CUDA sources include <glm/...>, a third-party header-only
// library that is not part of the reference tree and not installed on the build machine. To compile the
// reference's own, unmodified kernels as the comparator / parity pin, this directory supplies the names
// they use, written from the mathematical definitions (column-major matrices, Hamilton quaternions with
// a (w, x, y, z) constructor, shortest-arc slerp). Nothing of the product includes these files.
//
// Conventions that matter to the callers:
//   * mat<C, R, T> has C columns of R rows; m[i] is column i; the scalar-list constructor fills column
//     by column; mat(s) is s times the identity.
//   * vec / mat / qua are plain aggregates of T with alignment of T (so float arrays may be viewed
//     as arrays of vec3 / vec4 / mat3).
//   * T{} zero-initialises; a default-constructed object is uninitialised.
#pragma once

#include <cmath>
#include <cstddef>

#if defined(__CUDACC__)
#define GLMS_FN __host__ __device__ inline
#else
#define GLMS_FN inline
#endif

namespace glm {

    typedef int length_t;
    enum qualifier { packed_highp,
                     defaultp = packed_highp };

    template <length_t L, typename T, qualifier Q = defaultp>
    struct vec;
    template <length_t C, length_t R, typename T, qualifier Q = defaultp>
    struct mat;
    template <typename T, qualifier Q = defaultp>
    struct qua;

    // ------------------------------------------------------------------ vectors
    template <typename T, qualifier Q>
    struct vec<2, T, Q> {
        T x, y;
        vec() = default;
        GLMS_FN vec(T a, T b) : x(a), y(b) {}
        GLMS_FN explicit vec(T s) : x(s), y(s) {}
        template <typename U, qualifier P>
        GLMS_FN vec(const vec<2, U, P>& v) : x(T(v.x)), y(T(v.y)) {}
        template <typename U, qualifier P>
        GLMS_FN explicit vec(const vec<3, U, P>& v) : x(T(v.x)), y(T(v.y)) {}
        GLMS_FN T& operator[](length_t i) { return (&x)[i]; }
        GLMS_FN const T& operator[](length_t i) const { return (&x)[i]; }
        static GLMS_FN constexpr length_t length() { return 2; }
    };

    template <typename T, qualifier Q>
    struct vec<3, T, Q> {
        T x, y, z;
        vec() = default;
        GLMS_FN vec(T a, T b, T c) : x(a), y(b), z(c) {}
        GLMS_FN explicit vec(T s) : x(s), y(s), z(s) {}
        template <typename U, qualifier P>
        GLMS_FN vec(const vec<3, U, P>& v) : x(T(v.x)), y(T(v.y)), z(T(v.z)) {}
        GLMS_FN vec(const vec<2, T, Q>& v, T c) : x(v.x), y(v.y), z(c) {}
        template <qualifier P>
        GLMS_FN explicit vec(const vec<4, T, P>& v) : x(v.x), y(v.y), z(v.z) {}
        GLMS_FN T& operator[](length_t i) { return (&x)[i]; }
        GLMS_FN const T& operator[](length_t i) const { return (&x)[i]; }
        static GLMS_FN constexpr length_t length() { return 3; }
    };

    template <typename T, qualifier Q>
    struct vec<4, T, Q> {
        T x, y, z, w;
        vec() = default;
        GLMS_FN vec(T a, T b, T c, T d) : x(a), y(b), z(c), w(d) {}
        GLMS_FN explicit vec(T s) : x(s), y(s), z(s), w(s) {}
        template <typename U, qualifier P>
        GLMS_FN vec(const vec<4, U, P>& v) : x(T(v.x)), y(T(v.y)), z(T(v.z)), w(T(v.w)) {}
        GLMS_FN vec(const vec<3, T, Q>& v, T d) : x(v.x), y(v.y), z(v.z), w(d) {}
        GLMS_FN T& operator[](length_t i) { return (&x)[i]; }
        GLMS_FN const T& operator[](length_t i) const { return (&x)[i]; }
        static GLMS_FN constexpr length_t length() { return 4; }
    };

#define GLMS_VEC_BINOP(OP)                                                                      \
    template <length_t L, typename T, qualifier Q>                                              \
    GLMS_FN vec<L, T, Q> operator OP(const vec<L, T, Q>& a, const vec<L, T, Q>& b) {            \
        vec<L, T, Q> r;                                                                         \
        for (length_t i = 0; i < L; ++i)                                                        \
            r[i] = a[i] OP b[i];                                                                \
        return r;                                                                               \
    }                                                                                           \
    template <length_t L, typename T, qualifier Q>                                              \
    GLMS_FN vec<L, T, Q> operator OP(const vec<L, T, Q>& a, T s) {                              \
        vec<L, T, Q> r;                                                                         \
        for (length_t i = 0; i < L; ++i)                                                        \
            r[i] = a[i] OP s;                                                                   \
        return r;                                                                               \
    }                                                                                           \
    template <length_t L, typename T, qualifier Q>                                              \
    GLMS_FN vec<L, T, Q> operator OP(T s, const vec<L, T, Q>& b) {                              \
        vec<L, T, Q> r;                                                                         \
        for (length_t i = 0; i < L; ++i)                                                        \
            r[i] = s OP b[i];                                                                   \
        return r;                                                                               \
    }                                                                                           \
    template <length_t L, typename T, qualifier Q>                                              \
    GLMS_FN vec<L, T, Q>& operator OP##=(vec<L, T, Q>& a, const vec<L, T, Q>& b) {              \
        for (length_t i = 0; i < L; ++i)                                                        \
            a[i] OP## = b[i];                                                                   \
        return a;                                                                               \
    }                                                                                           \
    template <length_t L, typename T, qualifier Q>                                              \
    GLMS_FN vec<L, T, Q>& operator OP##=(vec<L, T, Q>& a, T s) {                                \
        for (length_t i = 0; i < L; ++i)                                                        \
            a[i] OP## = s;                                                                      \
        return a;                                                                               \
    }
    GLMS_VEC_BINOP(+)
    GLMS_VEC_BINOP(-)
    GLMS_VEC_BINOP(*)
    GLMS_VEC_BINOP(/)
#undef GLMS_VEC_BINOP

    template <length_t L, typename T, qualifier Q>
    GLMS_FN vec<L, T, Q> operator-(const vec<L, T, Q>& a) {
        vec<L, T, Q> r;
        for (length_t i = 0; i < L; ++i)
            r[i] = -a[i];
        return r;
    }
    template <length_t L, typename T, qualifier Q>
    GLMS_FN vec<L, T, Q> operator+(const vec<L, T, Q>& a) { return a; }
    template <length_t L, typename T, qualifier Q>
    GLMS_FN bool operator==(const vec<L, T, Q>& a, const vec<L, T, Q>& b) {
        bool e = true;
        for (length_t i = 0; i < L; ++i)
            e = e && (a[i] == b[i]);
        return e;
    }
    template <length_t L, typename T, qualifier Q>
    GLMS_FN bool operator!=(const vec<L, T, Q>& a, const vec<L, T, Q>& b) { return !(a == b); }

    // sum of products, accumulated left to right
    template <length_t L, typename T, qualifier Q>
    GLMS_FN T dot(const vec<L, T, Q>& a, const vec<L, T, Q>& b) {
        T s = a[0] * b[0];
        for (length_t i = 1; i < L; ++i)
            s = s + a[i] * b[i];
        return s;
    }
    template <typename T, qualifier Q>
    GLMS_FN vec<3, T, Q> cross(const vec<3, T, Q>& a, const vec<3, T, Q>& b) {
        return vec<3, T, Q>(a.y * b.z - b.y * a.z, a.z * b.x - b.z * a.x, a.x * b.y - b.x * a.y);
    }
    template <length_t L, typename T, qualifier Q>
    GLMS_FN T length(const vec<L, T, Q>& a) { return std::sqrt(dot(a, a)); }
    template <length_t L, typename T, qualifier Q>
    GLMS_FN vec<L, T, Q> normalize(const vec<L, T, Q>& a) { return a * (T(1) / std::sqrt(dot(a, a))); }

    // ------------------------------------------------------------------ matrices (column-major)
    template <length_t C, length_t R, typename T, qualifier Q>
    struct mat {
        typedef vec<R, T, Q> col_type;
        typedef vec<C, T, Q> row_type;
        col_type value[C];

        mat() = default;
        // s times the identity
        GLMS_FN explicit mat(T s) {
            for (length_t c = 0; c < C; ++c)
                for (length_t r = 0; r < R; ++r)
                    value[c][r] = (c == r) ? s : T(0);
        }
        // column by column
        GLMS_FN mat(T a0, T a1, T a2, T a3) {
            static_assert(C * R == 4, "4 scalars fill a 2x2 matrix");
            const T a[4] = {a0, a1, a2, a3};
            fill(a);
        }
        GLMS_FN mat(T a0, T a1, T a2, T a3, T a4, T a5) {
            static_assert(C * R == 6, "6 scalars fill a 3x2 or 2x3 matrix");
            const T a[6] = {a0, a1, a2, a3, a4, a5};
            fill(a);
        }
        GLMS_FN mat(T a0, T a1, T a2, T a3, T a4, T a5, T a6, T a7, T a8) {
            static_assert(C * R == 9, "9 scalars fill a 3x3 matrix");
            const T a[9] = {a0, a1, a2, a3, a4, a5, a6, a7, a8};
            fill(a);
        }
        GLMS_FN mat(T a0, T a1, T a2, T a3, T a4, T a5, T a6, T a7, T a8, T a9, T a10, T a11, T a12, T a13, T a14, T a15) {
            static_assert(C * R == 16, "16 scalars fill a 4x4 matrix");
            const T a[16] = {a0, a1, a2, a3, a4, a5, a6, a7, a8, a9, a10, a11, a12, a13, a14, a15};
            fill(a);
        }
        GLMS_FN mat(const col_type& c0, const col_type& c1) {
            static_assert(C == 2, "two columns");
            value[0] = c0;
            value[1] = c1;
        }
        GLMS_FN mat(const col_type& c0, const col_type& c1, const col_type& c2) {
            static_assert(C == 3, "three columns");
            value[0] = c0;
            value[1] = c1;
            value[2] = c2;
        }
        GLMS_FN col_type& operator[](length_t i) { return value[i]; }
        GLMS_FN const col_type& operator[](length_t i) const { return value[i]; }
        static GLMS_FN constexpr length_t length() { return C; }

    private:
        GLMS_FN void fill(const T* a) {
            for (length_t c = 0; c < C; ++c)
                for (length_t r = 0; r < R; ++r)
                    value[c][r] = a[c * R + r];
        }
    };

    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN mat<C, R, T, Q> operator+(const mat<C, R, T, Q>& a, const mat<C, R, T, Q>& b) {
        mat<C, R, T, Q> m;
        for (length_t c = 0; c < C; ++c)
            m[c] = a[c] + b[c];
        return m;
    }
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN mat<C, R, T, Q> operator-(const mat<C, R, T, Q>& a, const mat<C, R, T, Q>& b) {
        mat<C, R, T, Q> m;
        for (length_t c = 0; c < C; ++c)
            m[c] = a[c] - b[c];
        return m;
    }
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN mat<C, R, T, Q> operator-(const mat<C, R, T, Q>& a) {
        mat<C, R, T, Q> m;
        for (length_t c = 0; c < C; ++c)
            m[c] = -a[c];
        return m;
    }
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN mat<C, R, T, Q> operator*(const mat<C, R, T, Q>& a, T s) {
        mat<C, R, T, Q> m;
        for (length_t c = 0; c < C; ++c)
            m[c] = a[c] * s;
        return m;
    }
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN mat<C, R, T, Q> operator*(T s, const mat<C, R, T, Q>& a) {
        mat<C, R, T, Q> m;
        for (length_t c = 0; c < C; ++c)
            m[c] = s * a[c];
        return m;
    }
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN mat<C, R, T, Q> operator/(const mat<C, R, T, Q>& a, T s) {
        mat<C, R, T, Q> m;
        for (length_t c = 0; c < C; ++c)
            m[c] = a[c] / s;
        return m;
    }
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN mat<C, R, T, Q>& operator+=(mat<C, R, T, Q>& a, const mat<C, R, T, Q>& b) {
        for (length_t c = 0; c < C; ++c)
            a[c] += b[c];
        return a;
    }
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN mat<C, R, T, Q>& operator-=(mat<C, R, T, Q>& a, const mat<C, R, T, Q>& b) {
        for (length_t c = 0; c < C; ++c)
            a[c] -= b[c];
        return a;
    }
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN mat<C, R, T, Q>& operator*=(mat<C, R, T, Q>& a, T s) {
        for (length_t c = 0; c < C; ++c)
            a[c] *= s;
        return a;
    }
    // matrix times column vector: linear combination of the columns, left to right
    // (the vector's type is taken from the matrix, so a vector of another scalar type converts implicitly)
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN vec<R, T, Q> operator*(const mat<C, R, T, Q>& m, const typename mat<C, R, T, Q>::row_type& v) {
        vec<R, T, Q> r = m[0] * v[0];
        for (length_t c = 1; c < C; ++c)
            r = r + m[c] * v[c];
        return r;
    }
    // row vector times matrix
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN vec<C, T, Q> operator*(const typename mat<C, R, T, Q>::col_type& v, const mat<C, R, T, Q>& m) {
        vec<C, T, Q> r;
        for (length_t c = 0; c < C; ++c)
            r[c] = dot(v, m[c]);
        return r;
    }
    // (K columns of R rows) times (C columns of K rows) -> C columns of R rows
    template <length_t K, length_t R, length_t C, typename T, qualifier Q>
    GLMS_FN mat<C, R, T, Q> operator*(const mat<K, R, T, Q>& a, const mat<C, K, T, Q>& b) {
        mat<C, R, T, Q> m;
        for (length_t c = 0; c < C; ++c)
            m[c] = a * b[c];
        return m;
    }

    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN mat<R, C, T, Q> transpose(const mat<C, R, T, Q>& a) {
        mat<R, C, T, Q> m;
        for (length_t c = 0; c < C; ++c)
            for (length_t r = 0; r < R; ++r)
                m[r][c] = a[c][r];
        return m;
    }
    template <typename T, qualifier Q>
    GLMS_FN T determinant(const mat<2, 2, T, Q>& m) { return m[0][0] * m[1][1] - m[1][0] * m[0][1]; }
    template <typename T, qualifier Q>
    GLMS_FN T determinant(const mat<3, 3, T, Q>& m) {
        return m[0][0] * (m[1][1] * m[2][2] - m[2][1] * m[1][2]) - m[1][0] * (m[0][1] * m[2][2] - m[2][1] * m[0][2]) +
               m[2][0] * (m[0][1] * m[1][2] - m[1][1] * m[0][2]);
    }
    // adjugate times the reciprocal determinant
    template <typename T, qualifier Q>
    GLMS_FN mat<2, 2, T, Q> inverse(const mat<2, 2, T, Q>& m) {
        const T inv_det = T(1) / (m[0][0] * m[1][1] - m[1][0] * m[0][1]);
        return mat<2, 2, T, Q>(m[1][1] * inv_det, -m[0][1] * inv_det, -m[1][0] * inv_det, m[0][0] * inv_det);
    }
    template <typename T, qualifier Q>
    GLMS_FN mat<3, 3, T, Q> inverse(const mat<3, 3, T, Q>& m) {
        const T inv_det = T(1) / determinant(m);
        mat<3, 3, T, Q> r;
        r[0][0] = +(m[1][1] * m[2][2] - m[2][1] * m[1][2]) * inv_det;
        r[1][0] = -(m[1][0] * m[2][2] - m[2][0] * m[1][2]) * inv_det;
        r[2][0] = +(m[1][0] * m[2][1] - m[2][0] * m[1][1]) * inv_det;
        r[0][1] = -(m[0][1] * m[2][2] - m[2][1] * m[0][2]) * inv_det;
        r[1][1] = +(m[0][0] * m[2][2] - m[2][0] * m[0][2]) * inv_det;
        r[2][1] = -(m[0][0] * m[2][1] - m[2][0] * m[0][1]) * inv_det;
        r[0][2] = +(m[0][1] * m[1][2] - m[1][1] * m[0][2]) * inv_det;
        r[1][2] = -(m[0][0] * m[1][2] - m[1][0] * m[0][2]) * inv_det;
        r[2][2] = +(m[0][0] * m[1][1] - m[1][0] * m[0][1]) * inv_det;
        return r;
    }
    // column c times row r: result[j] = c * r[j], an R x C matrix for c in R^R, r in R^C
    template <length_t DA, length_t DB, typename T, qualifier Q>
    GLMS_FN mat<DB, DA, T, Q> outerProduct(const vec<DA, T, Q>& c, const vec<DB, T, Q>& r) {
        mat<DB, DA, T, Q> m;
        for (length_t j = 0; j < DB; ++j)
            m[j] = c * r[j];
        return m;
    }

    // ------------------------------------------------------------------ quaternions
    template <typename T, qualifier Q>
    struct qua {
        T x, y, z, w;
        qua() = default;
        // scalar part first
        GLMS_FN qua(T w_, T x_, T y_, T z_) : x(x_), y(y_), z(z_), w(w_) {}
        GLMS_FN qua(T s, const vec<3, T, Q>& v) : x(v.x), y(v.y), z(v.z), w(s) {}
        static GLMS_FN constexpr length_t length() { return 4; }
    };

    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> operator-(const qua<T, Q>& q) { return qua<T, Q>(-q.w, -q.x, -q.y, -q.z); }
    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> operator+(const qua<T, Q>& a, const qua<T, Q>& b) {
        return qua<T, Q>(a.w + b.w, a.x + b.x, a.y + b.y, a.z + b.z);
    }
    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> operator*(const qua<T, Q>& q, T s) { return qua<T, Q>(q.w * s, q.x * s, q.y * s, q.z * s); }
    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> operator*(T s, const qua<T, Q>& q) { return q * s; }
    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> operator/(const qua<T, Q>& q, T s) { return qua<T, Q>(q.w / s, q.x / s, q.y / s, q.z / s); }
    // Hamilton product
    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> operator*(const qua<T, Q>& p, const qua<T, Q>& q) {
        return qua<T, Q>(
            p.w * q.w - p.x * q.x - p.y * q.y - p.z * q.z,
            p.w * q.x + p.x * q.w + p.y * q.z - p.z * q.y,
            p.w * q.y + p.y * q.w + p.z * q.x - p.x * q.z,
            p.w * q.z + p.z * q.w + p.x * q.y - p.y * q.x);
    }
    // rotation of v by the unit quaternion q:  v + 2 (w (u x v) + u x (u x v)),  u = (x, y, z)
    template <typename T, qualifier Q>
    GLMS_FN vec<3, T, Q> operator*(const qua<T, Q>& q, const vec<3, T, Q>& v) {
        const vec<3, T, Q> u(q.x, q.y, q.z);
        const vec<3, T, Q> uv = cross(u, v);
        const vec<3, T, Q> uuv = cross(u, uv);
        return v + ((uv * q.w) + uuv) * T(2);
    }
    template <typename T, qualifier Q>
    GLMS_FN T dot(const qua<T, Q>& a, const qua<T, Q>& b) {
        return (a.x * b.x + a.y * b.y) + (a.z * b.z + a.w * b.w);
    }
    template <typename T, qualifier Q>
    GLMS_FN T length(const qua<T, Q>& q) { return std::sqrt(dot(q, q)); }
    // identity for a zero quaternion
    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> normalize(const qua<T, Q>& q) {
        const T len = length(q);
        if (len <= T(0))
            return qua<T, Q>(T(1), T(0), T(0), T(0));
        const T inv = T(1) / len;
        return qua<T, Q>(q.w * inv, q.x * inv, q.y * inv, q.z * inv);
    }
    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> conjugate(const qua<T, Q>& q) { return qua<T, Q>(q.w, -q.x, -q.y, -q.z); }
    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> inverse(const qua<T, Q>& q) { return conjugate(q) / dot(q, q); }
    template <typename T, qualifier Q>
    GLMS_FN vec<3, T, Q> rotate(const qua<T, Q>& q, const vec<3, T, Q>& v) { return q * v; }

    // rotation matrix of a unit quaternion
    template <typename T, qualifier Q>
    GLMS_FN mat<3, 3, T, Q> mat3_cast(const qua<T, Q>& q) {
        const T xx = q.x * q.x, yy = q.y * q.y, zz = q.z * q.z;
        const T xz = q.x * q.z, xy = q.x * q.y, yz = q.y * q.z;
        const T wx = q.w * q.x, wy = q.w * q.y, wz = q.w * q.z;
        mat<3, 3, T, Q> m;
        m[0][0] = T(1) - T(2) * (yy + zz);
        m[0][1] = T(2) * (xy + wz);
        m[0][2] = T(2) * (xz - wy);
        m[1][0] = T(2) * (xy - wz);
        m[1][1] = T(1) - T(2) * (xx + zz);
        m[1][2] = T(2) * (yz + wx);
        m[2][0] = T(2) * (xz + wy);
        m[2][1] = T(2) * (yz - wx);
        m[2][2] = T(1) - T(2) * (xx + yy);
        return m;
    }
    // quaternion of a rotation matrix: recover the component of largest magnitude from the diagonal,
    // the other three from the off-diagonal sums / differences
    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> quat_cast(const mat<3, 3, T, Q>& m) {
        const T four_x2_m1 = m[0][0] - m[1][1] - m[2][2];
        const T four_y2_m1 = m[1][1] - m[0][0] - m[2][2];
        const T four_z2_m1 = m[2][2] - m[0][0] - m[1][1];
        const T four_w2_m1 = m[0][0] + m[1][1] + m[2][2];
        int biggest = 0;
        T big = four_w2_m1;
        if (four_x2_m1 > big) {
            big = four_x2_m1;
            biggest = 1;
        }
        if (four_y2_m1 > big) {
            big = four_y2_m1;
            biggest = 2;
        }
        if (four_z2_m1 > big) {
            big = four_z2_m1;
            biggest = 3;
        }
        const T val = std::sqrt(big + T(1)) * T(0.5);
        const T mult = T(0.25) / val;
        switch (biggest) {
        case 0: return qua<T, Q>(val, (m[1][2] - m[2][1]) * mult, (m[2][0] - m[0][2]) * mult, (m[0][1] - m[1][0]) * mult);
        case 1: return qua<T, Q>((m[1][2] - m[2][1]) * mult, val, (m[0][1] + m[1][0]) * mult, (m[2][0] + m[0][2]) * mult);
        case 2: return qua<T, Q>((m[2][0] - m[0][2]) * mult, (m[0][1] + m[1][0]) * mult, val, (m[1][2] + m[2][1]) * mult);
        default: return qua<T, Q>((m[0][1] - m[1][0]) * mult, (m[2][0] + m[0][2]) * mult, (m[1][2] + m[2][1]) * mult, val);
        }
    }
    // spherical interpolation along the shortest arc; linear blend when the ends (almost) coincide
    template <typename T, qualifier Q>
    GLMS_FN qua<T, Q> slerp(const qua<T, Q>& a, const qua<T, Q>& b, T t) {
        qua<T, Q> c = b;
        T cos_theta = dot(a, b);
        if (cos_theta < T(0)) {
            c = -b;
            cos_theta = -cos_theta;
        }
        if (cos_theta > T(1) - T(1.1920928955078125e-07)) {
            return qua<T, Q>(a.w + t * (c.w - a.w), a.x + t * (c.x - a.x), a.y + t * (c.y - a.y), a.z + t * (c.z - a.z));
        }
        const T angle = std::acos(cos_theta);
        return (std::sin((T(1) - t) * angle) * a + std::sin(t * angle) * c) / std::sin(angle);
    }

    // Tait-Bryan angles (rotation about x, y, z) of a unit quaternion
    template <typename T, qualifier Q>
    GLMS_FN vec<3, T, Q> eulerAngles(const qua<T, Q>& q) {
        const T pitch = std::atan2(T(2) * (q.y * q.z + q.w * q.x), q.w * q.w - q.x * q.x - q.y * q.y + q.z * q.z);
        T s = T(-2) * (q.x * q.z - q.w * q.y);
        s = s < T(-1) ? T(-1) : (s > T(1) ? T(1) : s);
        const T yaw = std::asin(s);
        const T roll = std::atan2(T(2) * (q.x * q.y + q.w * q.z), q.w * q.w + q.x * q.x - q.y * q.y - q.z * q.z);
        return vec<3, T, Q>(pitch, yaw, roll);
    }

    // ------------------------------------------------------------------ pointer helpers
    template <typename T>
    GLMS_FN vec<2, T> make_vec2(const T* p) { return vec<2, T>(p[0], p[1]); }
    template <typename T>
    GLMS_FN vec<3, T> make_vec3(const T* p) { return vec<3, T>(p[0], p[1], p[2]); }
    template <typename T>
    GLMS_FN vec<4, T> make_vec4(const T* p) { return vec<4, T>(p[0], p[1], p[2], p[3]); }
    template <length_t L, typename T, qualifier Q>
    GLMS_FN const T* value_ptr(const vec<L, T, Q>& v) { return &v.x; }
    template <length_t L, typename T, qualifier Q>
    GLMS_FN T* value_ptr(vec<L, T, Q>& v) { return &v.x; }
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN const T* value_ptr(const mat<C, R, T, Q>& m) { return &m[0].x; }
    template <length_t C, length_t R, typename T, qualifier Q>
    GLMS_FN T* value_ptr(mat<C, R, T, Q>& m) { return &m[0].x; }

    // ------------------------------------------------------------------ the usual aliases
    typedef vec<2, float> vec2;
    typedef vec<3, float> vec3;
    typedef vec<4, float> vec4;
    typedef vec<2, float> fvec2;
    typedef vec<3, float> fvec3;
    typedef vec<4, float> fvec4;
    typedef mat<2, 2, float> mat2;
    typedef mat<3, 3, float> mat3;
    typedef mat<4, 4, float> mat4;
    typedef mat<2, 2, float> fmat2;
    typedef mat<3, 3, float> fmat3;
    typedef mat<4, 4, float> fmat4;
    typedef mat<3, 2, float> mat3x2;
    typedef mat<2, 3, float> mat2x3;
    typedef qua<float> quat;
    typedef qua<float> fquat;

} // namespace glm
