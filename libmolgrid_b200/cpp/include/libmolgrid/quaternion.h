// Float quaternion with the operation order of the reference class
// (include/libmolgrid/quaternion.h): products term by term, left to right, in single precision.
// Build host code with -ffp-contract=off so that no multiply-add is fused.
#ifndef LMGB200_QUATERNION_H_
#define LMGB200_QUATERNION_H_

#include "libmolgrid/common.h"

namespace libmolgrid {

class Quaternion {
  float a, b, c, d;  // real part, then i, j, k

 public:
  Quaternion() : a(1), b(0), c(0), d(0) {}
  Quaternion(float A, float B, float C, float D) : a(A), b(B), c(C), d(D) {}

  float R_component_1() const { return a; }
  float R_component_2() const { return b; }
  float R_component_3() const { return c; }
  float R_component_4() const { return d; }
  float real() const { return a; }

  Quaternion conj() const { return Quaternion(a, -b, -c, -d); }
  // squared Euclidean length
  float norm() const { return a * a + b * b + c * c + d * d; }
  Quaternion inverse() const {
    float n = a * a + b * b + c * c + d * d;
    return Quaternion(a / n, -b / n, -c / n, -d / n);
  }

  Quaternion operator*(const Quaternion& r) const {
    return Quaternion(a * r.a - b * r.b - c * r.c - d * r.d, a * r.b + b * r.a + c * r.d - d * r.c,
                      a * r.c - b * r.d + c * r.a + d * r.b, a * r.d + b * r.c - c * r.b + d * r.a);
  }
  Quaternion& operator*=(const Quaternion& r) { return *this = *this * r; }
  Quaternion operator/(float s) const { return Quaternion(a / s, b / s, c / s, d / s); }
  Quaternion operator/(const Quaternion& r) const {
    float den = r.a * r.a + r.b * r.b + r.c * r.c + r.d * r.d;
    return Quaternion((a * r.a + b * r.b + c * r.c + d * r.d) / den, (-a * r.b + b * r.a - c * r.d + d * r.c) / den,
                      (-a * r.c + b * r.d + c * r.a - d * r.b) / den, (-a * r.d - b * r.c + c * r.b + d * r.a) / den);
  }
  Quaternion& operator/=(const Quaternion& r) { return *this = *this / r; }
  bool operator==(const Quaternion& r) const { return a == r.a && b == r.b && c == r.c && d == r.d; }

  // this * (0,x,y,z) * (conj / norm)
  float3 rotate(float x, float y, float z) const {
    Quaternion p = *this * Quaternion(0, x, y, z) * (conj() / norm());
    return make_float3(p.b, p.c, p.d);
  }
  // rotate about `center`, then translate
  float3 transform(float x, float y, float z, float3 center, float3 translate) const {
    float3 p = rotate(x - center.x, y - center.y, z - center.z);
    return make_float3(p.x + center.x + translate.x, p.y + center.y + translate.y, p.z + center.z + translate.z);
  }
};

}  // namespace libmolgrid
#endif
