// Test infrastructure (oracle build only; never linked into the product library).
//
// CPU restatement of the part of the sphericart library
// (https://github.com/lab-cosmo/sphericart, an un-vendored git submodule of the reference,
// .gitmodules:13-15, pinned commit unknown) that the reference evaluator calls:
//
//   sphericart::SphericalHarmonics<double> sh(l_max);
//   sh.compute(xyz, sph);                             // spherical_harmonic.cpp:58-61
//   sh.compute_with_gradients(xyz, sph, dsph);        // mace.cpp:132-133
//
// Published definition restated here: orthonormal real spherical harmonics of the
// DIRECTION of each input vector (Y_00 = 1/(2 sqrt(pi))), ordered lm = l*l + l + m, with
//   m > 0 :  sqrt(2) N_lm Q_l^m(z) Re (x + i y)^m
//   m = 0 :           N_l0 Q_l^0(z)
//   m < 0 :  sqrt(2) N_l|m| Q_l^|m|(z) Im (x + i y)^|m|
// on the unit sphere, where Q_l^m = d^m P_l / dz^m (no Condon-Shortley phase) and
// N_lm = sqrt((2l+1)/(4 pi) (l-m)!/(l+m)!). This is the sign convention that the
// reference's own closed forms pin (libsymmetrix/source/spherical_harmonic.cpp:28-36 for
// real_sph_harm and :45-55 for the real<->complex relation used with sphericart).
// Layouts: sph[i*nlm + lm]; dsph[(i*3 + c)*nlm + lm] = d sph[i,lm] / d xyz[i,c].
#pragma once

#include <cmath>
#include <vector>

namespace sphericart {

template <typename T>
class SphericalHarmonics {
public:
    explicit SphericalHarmonics(size_t l_max) : l_max_(static_cast<int>(l_max)) {
        const int L = l_max_;
        norm_.assign((L + 1) * (L + 1), 0.0);
        for (int l = 0; l <= L; ++l) {
            for (int m = 0; m <= l; ++m) {
                // (l-m)!/(l+m)! as a running product
                double ratio = 1.0;
                for (int q = l - m + 1; q <= l + m; ++q) ratio /= static_cast<double>(q);
                norm_[l * (L + 1) + m] = std::sqrt((2 * l + 1) / (4.0 * M_PI) * ratio);
            }
        }
    }

    void compute(const std::vector<T>& xyz, std::vector<T>& sph) {
        const size_t n = xyz.size() / 3;
        const int nlm = (l_max_ + 1) * (l_max_ + 1);
        sph.resize(n * nlm);
        std::vector<T> scratch(3 * nlm);
        for (size_t i = 0; i < n; ++i)
            one_point(&xyz[3 * i], &sph[i * nlm], scratch.data(), false);
    }

    void compute_with_gradients(const std::vector<T>& xyz, std::vector<T>& sph, std::vector<T>& dsph) {
        const size_t n = xyz.size() / 3;
        const int nlm = (l_max_ + 1) * (l_max_ + 1);
        sph.resize(n * nlm);
        dsph.resize(3 * n * nlm);
        for (size_t i = 0; i < n; ++i)
            one_point(&xyz[3 * i], &sph[i * nlm], &dsph[3 * i * nlm], true);
    }

private:
    int l_max_;
    std::vector<double> norm_;

    // Evaluate all harmonics (and optionally Cartesian gradients) of one vector.
    void one_point(const T* v, T* y, T* dy, bool with_grad) const {
        const int L = l_max_;
        const int nlm = (L + 1) * (L + 1);
        const double r = std::sqrt(double(v[0]) * v[0] + double(v[1]) * v[1] + double(v[2]) * v[2]);
        const double ux = v[0] / r, uy = v[1] / r, uz = v[2] / r;

        // c[m] + i s[m] = (ux + i uy)^m
        std::vector<double> c(L + 2, 0.0), s(L + 2, 0.0);
        c[0] = 1.0;
        for (int m = 1; m <= L + 1; ++m) {
            c[m] = c[m - 1] * ux - s[m - 1] * uy;
            s[m] = s[m - 1] * ux + c[m - 1] * uy;
        }
        // Q[l][m] = d^m P_l / dz^m at uz, for m up to l (zero beyond)
        const int W = L + 2;
        std::vector<double> Q((L + 1) * W, 0.0);
        for (int m = 0; m <= L; ++m) {
            double dfact = 1.0;  // (2m-1)!!
            for (int q = 2 * m - 1; q > 1; q -= 2) dfact *= q;
            Q[m * W + m] = dfact;
            if (m + 1 <= L) Q[(m + 1) * W + m] = (2 * m + 1) * uz * dfact;
            for (int l = m + 2; l <= L; ++l)
                Q[l * W + m] = ((2 * l - 1) * uz * Q[(l - 1) * W + m] - (l + m - 1) * Q[(l - 2) * W + m]) / (l - m);
        }

        std::vector<double> g(3 * nlm, 0.0);  // gradient w.r.t. the unit vector (polynomial extension)
        for (int l = 0; l <= L; ++l) {
            for (int m = 0; m <= l; ++m) {
                const double N = norm_[l * (L + 1) + m];
                const double q = Q[l * W + m];
                const double dq = (m + 1 <= l) ? Q[l * W + m + 1] : 0.0;  // dQ_l^m/dz = Q_l^{m+1}
                if (m == 0) {
                    const int lm = l * l + l;
                    y[lm] = static_cast<T>(N * q);
                    g[2 * nlm + lm] = N * dq;
                } else {
                    const double f = std::sqrt(2.0) * N;
                    const int lp = l * l + l + m, ln = l * l + l - m;
                    y[lp] = static_cast<T>(f * q * c[m]);
                    y[ln] = static_cast<T>(f * q * s[m]);
                    g[0 * nlm + lp] = f * q * m * c[m - 1];
                    g[1 * nlm + lp] = -f * q * m * s[m - 1];
                    g[2 * nlm + lp] = f * dq * c[m];
                    g[0 * nlm + ln] = f * q * m * s[m - 1];
                    g[1 * nlm + ln] = f * q * m * c[m - 1];
                    g[2 * nlm + ln] = f * dq * s[m];
                }
            }
        }
        if (!with_grad) return;
        // Chain rule through u = v/|v|: grad_v = (I - u u^T) grad_u / r
        for (int lm = 0; lm < nlm; ++lm) {
            const double gx = g[lm], gy = g[nlm + lm], gz = g[2 * nlm + lm];
            const double radial = gx * ux + gy * uy + gz * uz;
            dy[0 * nlm + lm] = static_cast<T>((gx - radial * ux) / r);
            dy[1 * nlm + lm] = static_cast<T>((gy - radial * uy) / r);
            dy[2 * nlm + lm] = static_cast<T>((gz - radial * uz) / r);
        }
    }
};

}  // namespace sphericart
