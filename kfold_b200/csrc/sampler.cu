// The coordinate-space steps of K-Fold's sampler loop around the score network (model/modules/ecsi.py:498-560): random
// rotation + translation of the coordinate sets, forward-pinned churn and input preconditioning, and -- in one kernel --
// output preconditioning, rotation-only rigid alignment, centring and the SI / ECSI update.
//
// A "coordinate set" is one diffusion sample of one complex: l atoms x 3 fp32 coordinates, contiguous.  The n sets of a
// call are ordered (complex, sample); `mask_div` consecutive sets (the samples of a complex) share one atom-mask row.
// Everything here is HBM-trivial (tens of KB per set); the point of these kernels is to replace the dozens of tiny
// element-wise and reduction launches the torch formulation needs per sampler step by three.
#include "ops_common.cuh"

using namespace kfb;

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sums `K` per-thread partials over the block; every thread gets the totals.  `scratch`: K * 8 doubles of shared memory.
template <int K>
__device__ __forceinline__ void block_sum(double (&v)[K], double* scratch) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();   // scratch may still be read from an earlier call
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const double s = warp_sum(v[k]);
    if (lane == 0) scratch[k * (kThreads / 32) + warp] = s;
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < K; ++k) {
    double s = 0.0;
#pragma unroll
    for (int w = 0; w < kThreads / 32; ++w) s += scratch[k * (kThreads / 32) + w];
    v[k] = s;
  }
}

// Rotation of a quaternion built from four standard normals o: q = o / copysign(|o|, o0), R as in
// utils/geometry/random_augment.py:296-350 (real part first; R applied to row vectors: out[s] = sum_d x[d] R[d][s]).
__device__ __forceinline__ void rotation_from_normals(const float* o, float (&R)[9]) {
  const float s = o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3];
  const float nrm = copysignf(sqrtf(s), o[0]);
  const float r = o[0] / nrm, i = o[1] / nrm, j = o[2] / nrm, k = o[3] / nrm;
  const float two_s = 2.0f / (r * r + i * i + j * j + k * k);
  R[0] = 1.f - two_s * (j * j + k * k); R[1] = two_s * (i * j - k * r);       R[2] = two_s * (i * k + j * r);
  R[3] = two_s * (i * j + k * r);       R[4] = 1.f - two_s * (i * i + k * k); R[5] = two_s * (j * k - i * r);
  R[6] = two_s * (i * k - j * r);       R[7] = two_s * (j * k + i * r);       R[8] = 1.f - two_s * (i * i + j * j);
}

__global__ void __launch_bounds__(kThreads) coords_augment_kernel(float* __restrict__ xa, float* __restrict__ xb,
                                                                  const float* __restrict__ normals, const float* __restrict__ trans,
                                                                  const unsigned char* __restrict__ mask, int l, int mask_div) {
  const int set = blockIdx.x;
  float R[9];
  rotation_from_normals(normals + 4 * set, R);
  const float t0 = trans ? trans[3 * set] : 0.f, t1 = trans ? trans[3 * set + 1] : 0.f, t2 = trans ? trans[3 * set + 2] : 0.f;
  const unsigned char* m = mask + static_cast<long long>(set / mask_div) * l;
  for (int a = threadIdx.x; a < l; a += kThreads) {
    const bool keep = m[a] != 0;
    for (int which = 0; which < 2; ++which) {
      float* x = which == 0 ? xa : xb;
      if (x == nullptr) continue;
      float* p = x + (static_cast<long long>(set) * l + a) * 3;
      const float x0 = p[0], x1 = p[1], x2 = p[2];
      p[0] = keep ? x0 * R[0] + x1 * R[3] + x2 * R[6] + t0 : 0.f;
      p[1] = keep ? x0 * R[1] + x1 * R[4] + x2 * R[7] + t1 : 0.f;
      p[2] = keep ? x0 * R[2] + x1 * R[5] + x2 * R[8] + t2 : 0.f;
    }
  }
}

// x_hat = a x_t + b x_T + c noise (noise zero on padding atoms); r6 = [c_in x_hat | x_T / sigma_T]
__global__ void __launch_bounds__(kThreads) sampler_prepare_kernel(const float* __restrict__ xt, const float* __restrict__ xT,
                                                                   const float* __restrict__ noise, const unsigned char* __restrict__ mask,
                                                                   float a, float b, float c, float c_in, float inv_sigma_T,
                                                                   float* __restrict__ x_hat, float* __restrict__ r6, long long atoms,
                                                                   int l, int mask_div) {
  const long long i = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= atoms) return;
  const long long set = i / l;
  const bool keep = mask[(set / mask_div) * l + (i - set * l)] != 0;
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    const float vt = xt[i * 3 + d], vT = xT[i * 3 + d];
    float v = a * vt + b * vT;
    if (noise != nullptr && keep) v += c * noise[i * 3 + d];
    if (noise == nullptr) v = vt;          // no churn at this step: the coordinates pass through unchanged
    x_hat[i * 3 + d] = v;
    r6[i * 6 + d] = c_in * v;
    r6[i * 6 + 3 + d] = vT * inv_sigma_T;
  }
}

// Largest eigenvector of a symmetric 4 x 4 matrix by cyclic Jacobi rotations (double precision).
__device__ void max_eigenvector4(double (&A)[4][4], double (&q)[4]) {
  double V[4][4] = {{1, 0, 0, 0}, {0, 1, 0, 0}, {0, 0, 1, 0}, {0, 0, 0, 1}};
  for (int sweep = 0; sweep < 16; ++sweep) {
    double off = 0.0;
    for (int p = 0; p < 3; ++p)
      for (int r = p + 1; r < 4; ++r) off += A[p][r] * A[p][r];
    if (off < 1e-280) break;
    for (int p = 0; p < 3; ++p) {
      for (int r = p + 1; r < 4; ++r) {
        if (fabs(A[p][r]) < 1e-300) continue;
        const double theta = (A[r][r] - A[p][p]) / (2.0 * A[p][r]);
        const double t = (theta >= 0.0 ? 1.0 : -1.0) / (fabs(theta) + sqrt(theta * theta + 1.0));
        const double c = 1.0 / sqrt(t * t + 1.0), s = t * c;
        for (int k = 0; k < 4; ++k) {
          const double akp = A[k][p], akr = A[k][r];
          A[k][p] = c * akp - s * akr;
          A[k][r] = s * akp + c * akr;
        }
        for (int k = 0; k < 4; ++k) {
          const double apk = A[p][k], ark = A[r][k];
          A[p][k] = c * apk - s * ark;
          A[r][k] = s * apk + c * ark;
        }
        for (int k = 0; k < 4; ++k) {
          const double vkp = V[k][p], vkr = V[k][r];
          V[k][p] = c * vkp - s * vkr;
          V[k][r] = s * vkp + c * vkr;
        }
      }
    }
  }
  int best = 0;
  for (int k = 1; k < 4; ++k)
    if (A[k][k] > A[best][best]) best = k;
  double n = 0.0;
  for (int k = 0; k < 4; ++k) n += V[k][best] * V[k][best];
  n = n > 0.0 ? 1.0 / sqrt(n) : 0.0;
  for (int k = 0; k < 4; ++k) q[k] = V[k][best] * n;
  if (n == 0.0) { q[0] = 1.0; q[1] = q[2] = q[3] = 0.0; }
}

// The proper rotation that best maps the (weighted, centred) coordinates c onto the targets t in the least-squares
// sense, from their covariance M[i][j] = sum_n w c_i t_j: Horn's quaternion form of the Kabsch problem -- the largest
// eigenvector of a symmetric 4 x 4 matrix is the rotation's quaternion, reflections cannot occur.  It equals the
// reference's U diag(1, 1, det) V^T from the SVD of M (utils/geometry/rigid_align.py:742-758) wherever that is unique.
// Result RT (row-vector form): aligned[s] = sum_d c[d] RT[d * 3 + s].
__device__ void kabsch_rotation(const double (&M)[9], float* RT) {
  const double Sxx = M[0], Sxy = M[1], Sxz = M[2], Syx = M[3], Syy = M[4], Syz = M[5], Szx = M[6], Szy = M[7], Szz = M[8];
  double N[4][4] = {{Sxx + Syy + Szz, Syz - Szy, Szx - Sxz, Sxy - Syx},
                    {Syz - Szy, Sxx - Syy - Szz, Sxy + Syx, Szx + Sxz},
                    {Szx - Sxz, Sxy + Syx, -Sxx + Syy - Szz, Syz + Szy},
                    {Sxy - Syx, Szx + Sxz, Syz + Szy, -Sxx - Syy + Szz}};
  double q[4];
  max_eigenvector4(N, q);
  const double q0 = q[0], qx = q[1], qy = q[2], qz = q[3];
  const double R[9] = {q0 * q0 + qx * qx - qy * qy - qz * qz, 2 * (qx * qy - q0 * qz), 2 * (qx * qz + q0 * qy),
                       2 * (qy * qx + q0 * qz), q0 * q0 - qx * qx + qy * qy - qz * qz, 2 * (qy * qz - q0 * qx),
                       2 * (qz * qx - q0 * qy), 2 * (qz * qy + q0 * qx), q0 * q0 - qx * qx - qy * qy + qz * qz};
  for (int d = 0; d < 3; ++d)
    for (int s = 0; s < 3; ++s) RT[d * 3 + s] = static_cast<float>(R[s * 3 + d]);
}

// One block per coordinate set.  coords = c_skip * xa + c_out * xb when xb is given (the preconditioned network output),
// else xa; fitted onto `target` over the masked atoms.  Leaves in shared memory: RT[9], the weighted centroid of the
// coordinates cc[3], of the targets tc[3], and the atom count W.
struct FitResult {
  float RT[9];
  float cc[3], tc[3];
  float W;
};
__device__ void fit_rotation(const float* __restrict__ xa, const float* __restrict__ xb, float c_skip, float c_out,
                             const float* __restrict__ target, const unsigned char* __restrict__ m, int l, FitResult* res,
                             double* scratch) {
  auto coord = [&](int a, int d) -> float {
    const float v = xa[a * 3 + d];
    return xb != nullptr ? c_skip * v + c_out * xb[a * 3 + d] : v;
  };
  double s[7] = {0, 0, 0, 0, 0, 0, 0};
  for (int a = threadIdx.x; a < l; a += kThreads) {
    if (!m[a]) continue;
    s[0] += 1.0;
    for (int d = 0; d < 3; ++d) {
      s[1 + d] += coord(a, d);
      s[4 + d] += target[a * 3 + d];
    }
  }
  block_sum<7>(s, scratch);
  const double w_sum = s[0] + 1e-8;     // the reference's eps (utils/geometry/rigid_align.py:733)
  const double cc[3] = {s[1] / w_sum, s[2] / w_sum, s[3] / w_sum}, tc[3] = {s[4] / w_sum, s[5] / w_sum, s[6] / w_sum};
  double M[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  for (int a = threadIdx.x; a < l; a += kThreads) {
    if (!m[a]) continue;
    double c[3], t[3];
    for (int d = 0; d < 3; ++d) {
      c[d] = coord(a, d) - cc[d];
      t[d] = target[a * 3 + d] - tc[d];
    }
    for (int i = 0; i < 3; ++i)
      for (int j = 0; j < 3; ++j) M[i * 3 + j] += c[i] * t[j];
  }
  block_sum<9>(M, scratch);
  if (threadIdx.x == 0) {
    if (s[0] > 0.0) {
      kabsch_rotation(M, res->RT);
    } else {   // no atom to fit on: identity (utils/geometry/rigid_align.py:718-723)
      for (int i = 0; i < 9; ++i) res->RT[i] = (i % 4 == 0) ? 1.f : 0.f;
    }
    for (int d = 0; d < 3; ++d) {
      res->cc[d] = static_cast<float>(cc[d]);
      res->tc[d] = static_cast<float>(tc[d]);
    }
    res->W = static_cast<float>(s[0]);
  }
  __syncthreads();
}

// custom_rigid_align with output_mask = mask (model/modules/ecsi.py:59-103)
__global__ void __launch_bounds__(kThreads) rigid_align_kernel(const float* __restrict__ coords, const float* __restrict__ target,
                                                               const unsigned char* __restrict__ mask, int rotation_only,
                                                               float* __restrict__ out, int l, int mask_div) {
  __shared__ FitResult fit;
  __shared__ double scratch[9 * (kThreads / 32)];
  const int set = blockIdx.x;
  const unsigned char* m = mask + static_cast<long long>(set / mask_div) * l;
  const float* c = coords + static_cast<long long>(set) * l * 3;
  const float* t = target + static_cast<long long>(set) * l * 3;
  float* o = out + static_cast<long long>(set) * l * 3;
  fit_rotation(c, nullptr, 0.f, 0.f, t, m, l, &fit, scratch);
  // translation: target centre - coordinate centre * RT
  float T[3];
  for (int s = 0; s < 3; ++s)
    T[s] = rotation_only ? 0.f : fit.tc[s] - (fit.cc[0] * fit.RT[s] + fit.cc[1] * fit.RT[3 + s] + fit.cc[2] * fit.RT[6 + s]);
  for (int a = threadIdx.x; a < l; a += kThreads) {
    const bool keep = m[a] != 0;
    const float x0 = c[a * 3], x1 = c[a * 3 + 1], x2 = c[a * 3 + 2];
    for (int s = 0; s < 3; ++s)
      o[a * 3 + s] = keep ? x0 * fit.RT[s] + x1 * fit.RT[3 + s] + x2 * fit.RT[6 + s] + T[s] : 0.f;
  }
}

// do_centering with mask_to_zero (utils/geometry/random_augment.py:90-130)
__global__ void __launch_bounds__(kThreads) center_coords_kernel(const float* __restrict__ coords, const unsigned char* __restrict__ mask,
                                                                 float* __restrict__ out, int l, int mask_div) {
  __shared__ double scratch[4 * (kThreads / 32)];
  const int set = blockIdx.x;
  const unsigned char* m = mask + static_cast<long long>(set / mask_div) * l;
  const float* c = coords + static_cast<long long>(set) * l * 3;
  float* o = out + static_cast<long long>(set) * l * 3;
  double s[4] = {0, 0, 0, 0};
  for (int a = threadIdx.x; a < l; a += kThreads) {
    if (!m[a]) continue;
    s[0] += 1.0;
    for (int d = 0; d < 3; ++d) s[1 + d] += c[a * 3 + d];
  }
  block_sum<4>(s, scratch);
  const double cnt = s[0] < 1.0 ? 1.0 : s[0];
  const bool any = s[0] > 0.0;       // an all-padding set is returned as it is (random_augment.py:110-112)
  for (int a = threadIdx.x; a < l; a += kThreads)
    for (int d = 0; d < 3; ++d)
      o[a * 3 + d] = !any ? c[a * 3 + d] : (m[a] ? c[a * 3 + d] - static_cast<float>(s[1 + d] / cnt) : 0.f);
}

// x0 = c_skip x_noisy + c_out r_update; rotated (rotation only) onto x_noisy over the valid atoms; centred; then
// x_next = ca x_noisy + cb x0 + cc x_T + cd noise (noise zero on padding atoms).  One block per coordinate set.
__global__ void __launch_bounds__(kThreads) sampler_update_kernel(const float* __restrict__ x_noisy, const float* __restrict__ r_update,
                                                                  const float* __restrict__ xT, const float* __restrict__ noise,
                                                                  const unsigned char* __restrict__ mask, float c_skip, float c_out,
                                                                  float ca, float cb, float cc_, float cd, float* __restrict__ x_next,
                                                                  float* __restrict__ x0_out, int l, int mask_div) {
  __shared__ FitResult fit;
  __shared__ double scratch[9 * (kThreads / 32)];
  const int set = blockIdx.x;
  const long long base = static_cast<long long>(set) * l * 3;
  const unsigned char* m = mask + static_cast<long long>(set / mask_div) * l;
  const float* xn = x_noisy + base;
  const float* ru = r_update + base;
  fit_rotation(xn, ru, c_skip, c_out, xn, m, l, &fit, scratch);
  // centre of the rotated, masked coordinates = (sum of the masked coordinates) RT / max(count, 1)
  const float scale = fit.W / fmaxf(fit.W, 1.f);     // (W + eps) cancels up to 1e-8 / W
  float ctr[3];
  for (int s = 0; s < 3; ++s) ctr[s] = scale * (fit.cc[0] * fit.RT[s] + fit.cc[1] * fit.RT[3 + s] + fit.cc[2] * fit.RT[6 + s]);
  for (int a = threadIdx.x; a < l; a += kThreads) {
    const bool keep = m[a] != 0;
    float x0[3];
    for (int d = 0; d < 3; ++d) x0[d] = c_skip * xn[a * 3 + d] + c_out * ru[a * 3 + d];
    for (int s = 0; s < 3; ++s) {
      const float al = keep ? x0[0] * fit.RT[s] + x0[1] * fit.RT[3 + s] + x0[2] * fit.RT[6 + s] - ctr[s] : 0.f;
      float v = ca * xn[a * 3 + s] + cb * al + cc_ * xT[base + a * 3 + s];
      if (noise != nullptr && keep) v += cd * noise[base + a * 3 + s];
      x_next[base + a * 3 + s] = v;
      if (x0_out != nullptr) x0_out[base + a * 3 + s] = al;
    }
  }
}

int check_sets(const char* what, int n, int l, int mask_div) {
  KFB_CHECK_ARG(n >= 1 && l >= 1 && mask_div >= 1 && n % mask_div == 0, "%s: %d coordinate sets of %d atoms, %d sets per mask row", what,
                n, l, mask_div);
  return KFB_OK;
}

}  // namespace

extern "C" {

KFB_API int kfb_coords_augment(float* x_a, float* x_b, const float* normals4, const float* trans, const unsigned char* mask, int n,
                               int l, int mask_div, void* stream_) {
  KFB_CHECK_ARG(x_a && normals4 && mask, "coords_augment: null pointer");
  KFB_TRY(check_sets("coords_augment", n, l, mask_div));
  cudaStream_t stream = as_stream(stream_);
  {
    LaunchScope scope(stream, "coords_augment");
    coords_augment_kernel<<<n, kThreads, 0, stream>>>(x_a, x_b, normals4, trans, mask, l, mask_div);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_sampler_prepare(const float* x_t, const float* x_T, const float* noise, const unsigned char* mask, float a, float b,
                                float c, float c_in, float inv_sigma_T, float* x_hat, float* r6, int n, int l, int mask_div,
                                void* stream_) {
  KFB_CHECK_ARG(x_t && x_T && mask && x_hat && r6, "sampler_prepare: null pointer");
  KFB_TRY(check_sets("sampler_prepare", n, l, mask_div));
  cudaStream_t stream = as_stream(stream_);
  const long long atoms = static_cast<long long>(n) * l;
  {
    LaunchScope scope(stream, "sampler_prepare");
    sampler_prepare_kernel<<<static_cast<unsigned>((atoms + kThreads - 1) / kThreads), kThreads, 0, stream>>>(
        x_t, x_T, noise, mask, a, b, c, c_in, inv_sigma_T, x_hat, r6, atoms, l, mask_div);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_sampler_update(const float* x_noisy, const float* r_update, const float* x_T, const float* noise,
                               const unsigned char* mask, float c_skip, float c_out, float ca, float cb, float cc, float cd,
                               float* x_next, float* x0_hat, int n, int l, int mask_div, void* stream_) {
  KFB_CHECK_ARG(x_noisy && r_update && x_T && mask && x_next, "sampler_update: null pointer");
  KFB_TRY(check_sets("sampler_update", n, l, mask_div));
  cudaStream_t stream = as_stream(stream_);
  {
    LaunchScope scope(stream, "sampler_update");
    sampler_update_kernel<<<n, kThreads, 0, stream>>>(x_noisy, r_update, x_T, noise, mask, c_skip, c_out, ca, cb, cc, cd, x_next,
                                                      x0_hat, l, mask_div);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_rigid_align(const float* coords, const float* target, const unsigned char* mask, int rotation_only, float* out, int n,
                            int l, int mask_div, void* stream_) {
  KFB_CHECK_ARG(coords && target && mask && out, "rigid_align: null pointer");
  KFB_TRY(check_sets("rigid_align", n, l, mask_div));
  cudaStream_t stream = as_stream(stream_);
  {
    LaunchScope scope(stream, "rigid_align");
    rigid_align_kernel<<<n, kThreads, 0, stream>>>(coords, target, mask, rotation_only, out, l, mask_div);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

KFB_API int kfb_center_coords(const float* coords, const unsigned char* mask, float* out, int n, int l, int mask_div, void* stream_) {
  KFB_CHECK_ARG(coords && mask && out, "center_coords: null pointer");
  KFB_TRY(check_sets("center_coords", n, l, mask_div));
  cudaStream_t stream = as_stream(stream_);
  {
    LaunchScope scope(stream, "center_coords");
    center_coords_kernel<<<n, kThreads, 0, stream>>>(coords, mask, out, l, mask_div);
  }
  KFB_CUDA(cudaGetLastError());
  return KFB_OK;
}

}  // extern "C"
