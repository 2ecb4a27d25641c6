// Stand-in for the un-vendored sphericart 1.0.3 dependency, used ONLY to build
// the reference's serial evaluator as a test oracle.  It provides the one class
// and the one method that evaluator calls (libsymmetrix/source/mace.cpp:1283-1284):
// orthonormal real spherical harmonics of the direction of each input vector,
// order lm = l*l + l + m, together with their Cartesian gradients.
//
// The arithmetic is an independent statement of the textbook formulas, not the
// dependency's source: every Y_lm is written as a homogeneous polynomial P_lm of
// degree l in the unit vector u, and the gradient with respect to the
// un-normalised input follows from Euler's theorem,
//     dY/dX = (grad P_lm(u) - l * P_lm(u) * u) / |X| .
// Layout of the outputs as the caller expects them: sph[n*size + lm] and
// dsph[n*3*size + d*size + lm].
#pragma once
#include <cmath>
#include <cstddef>
#include <stdexcept>
#include <vector>

namespace sphericart {

template <typename T>
class SphericalHarmonics {
public:
    explicit SphericalHarmonics(std::size_t l_max) : l_max_(static_cast<int>(l_max))
    {
        if (l_max_ < 0 || l_max_ > 3)
            throw std::invalid_argument("oracle sphericart stand-in supports l_max 0..3");
    }

    void compute_with_gradients(const std::vector<T>& xyz, std::vector<T>& sph, std::vector<T>& dsph)
    {
        const int size = (l_max_ + 1) * (l_max_ + 1);
        const std::size_t n = xyz.size() / 3;
        sph.resize(n * size);
        dsph.resize(n * 3 * size);
        for (std::size_t s = 0; s < n; ++s)
            sample(xyz.data() + 3 * s, sph.data() + s * size, dsph.data() + s * 3 * size, size);
    }

private:
    int l_max_;

    void sample(const T* v, T* y, T* g, int size) const
    {
        const double pi = 3.14159265358979323846;
        T p[16], gx[16], gy[16], gz[16];
        for (int i = 0; i < 16; ++i) p[i] = gx[i] = gy[i] = gz[i] = T(0);
        const T rr = v[0] * v[0] + v[1] * v[1] + v[2] * v[2];
        p[0] = static_cast<T>(0.5 * std::sqrt(1.0 / pi));
        if (rr == T(0)) {
            for (int i = 0; i < size; ++i) { y[i] = p[i]; g[i] = g[size + i] = g[2 * size + i] = T(0); }
            return;
        }
        const T inv = T(1) / std::sqrt(rr);
        const T x = v[0] * inv, yy = v[1] * inv, z = v[2] * inv;
        const T x2 = x * x, y2 = yy * yy, z2 = z * z;
        if (l_max_ >= 1) {
            const T c1 = static_cast<T>(std::sqrt(3.0 / (4.0 * pi)));
            p[1] = c1 * yy; gy[1] = c1;
            p[2] = c1 * z;  gz[2] = c1;
            p[3] = c1 * x;  gx[3] = c1;
        }
        if (l_max_ >= 2) {
            const T a = static_cast<T>(0.5 * std::sqrt(15.0 / pi));
            const T b = static_cast<T>(0.25 * std::sqrt(5.0 / pi));
            const T h = static_cast<T>(0.25 * std::sqrt(15.0 / pi));
            p[4] = a * x * yy;             gx[4] = a * yy;        gy[4] = a * x;
            p[5] = a * yy * z;             gy[5] = a * z;         gz[5] = a * yy;
            p[6] = b * (T(2) * z2 - x2 - y2);
            gx[6] = -T(2) * b * x;         gy[6] = -T(2) * b * yy; gz[6] = T(4) * b * z;
            p[7] = a * x * z;              gx[7] = a * z;         gz[7] = a * x;
            p[8] = h * (x2 - y2);          gx[8] = T(2) * h * x;  gy[8] = -T(2) * h * yy;
        }
        if (l_max_ >= 3) {
            const T c = static_cast<T>(0.25 * std::sqrt(35.0 / (2.0 * pi)));
            const T d = static_cast<T>(0.5 * std::sqrt(105.0 / pi));
            const T e = static_cast<T>(0.25 * std::sqrt(21.0 / (2.0 * pi)));
            const T f = static_cast<T>(0.25 * std::sqrt(7.0 / pi));
            const T k = static_cast<T>(0.25 * std::sqrt(105.0 / pi));
            const T q = T(4) * z2 - x2 - y2;
            p[9] = c * yy * (T(3) * x2 - y2);
            gx[9] = T(6) * c * x * yy;     gy[9] = T(3) * c * (x2 - y2);
            p[10] = d * x * yy * z;
            gx[10] = d * yy * z;           gy[10] = d * x * z;    gz[10] = d * x * yy;
            p[11] = e * yy * q;
            gx[11] = -T(2) * e * x * yy;   gy[11] = e * (q - T(2) * y2); gz[11] = T(8) * e * yy * z;
            p[12] = f * z * (T(2) * z2 - T(3) * x2 - T(3) * y2);
            gx[12] = -T(6) * f * x * z;    gy[12] = -T(6) * f * yy * z;
            gz[12] = f * (T(6) * z2 - T(3) * x2 - T(3) * y2);
            p[13] = e * x * q;
            gx[13] = e * (q - T(2) * x2);  gy[13] = -T(2) * e * x * yy; gz[13] = T(8) * e * x * z;
            p[14] = k * z * (x2 - y2);
            gx[14] = T(2) * k * x * z;     gy[14] = -T(2) * k * yy * z; gz[14] = k * (x2 - y2);
            p[15] = c * x * (x2 - T(3) * y2);
            gx[15] = T(3) * c * (x2 - y2); gy[15] = -T(6) * c * x * yy;
        }
        for (int lm = 0; lm < size; ++lm) {
            const int l = lm < 1 ? 0 : (lm < 4 ? 1 : (lm < 9 ? 2 : 3));
            const T radial = static_cast<T>(l) * p[lm];
            y[lm] = p[lm];
            g[lm] = (gx[lm] - x * radial) * inv;
            g[size + lm] = (gy[lm] - yy * radial) * inv;
            g[2 * size + lm] = (gz[lm] - z * radial) * inv;
        }
    }
};

}  // namespace sphericart
