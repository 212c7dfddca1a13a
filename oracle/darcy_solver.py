"""CPU oracle for the reference's Darcy data generator.  TEST INFRASTRUCTURE ONLY.

Restates dataset/darcy_generate/{Gaussian_Random_Field,Darcy_Gen,Solve_GWF}.m in numpy / scipy (float64, as MATLAB
computes): a thresholded Gaussian random field as the coefficient a(x), forcing f = 1, and the solution of
-div(a grad p) = f on [0,1]^2 with p = 0 on the boundary by a 5-point finite-volume scheme on the K x K node grid
after a cubic-spline resampling from cell centres to nodes and back.  Only tests may import it; the product's
generator (spgt_b200/dataset/darcy_generate.py) solves the same linear system with the library's CUDA solver.

Parity status: PARITY UNPINNED.  The reference's generator is MATLAB code, there is no MATLAB or Octave here and the
reference ships no generated sample, so this restatement could not be run against the original.  It is checked
instead by properties: the assembled operator is symmetric positive definite, the solution satisfies the discrete
equations, and for a = 1 it converges to the series solution of the Poisson problem on the unit square.
MATLAB's interp2(..., 'spline') is a tensor product of not-a-knot cubic splines; scipy's CubicSpline uses the same
end condition by default.
"""
from __future__ import annotations

import numpy as np


def gaussian_random_field(S: int, rng: np.random.Generator, alpha: float = 2.0, tau: float = 3.0) -> np.ndarray:
    """U = idct2(S * tau^(alpha-1) * (pi^2 |k|^2 + tau^2)^(-alpha/2) * N(0,1)), zero mean mode
    (Gaussian_Random_Field.m:10-19)."""
    import scipy.fft
    k1, k2 = np.meshgrid(np.arange(S), np.arange(S))
    coef = tau ** (alpha - 1) * (np.pi ** 2 * (k1 ** 2 + k2 ** 2) + tau ** 2) ** (-alpha / 2)
    L = S * coef * rng.standard_normal((S, S))
    L[0, 0] = 0.0
    return scipy.fft.idctn(L, type=2, norm='ortho')


def threshold_coefficient(U: np.ndarray) -> np.ndarray:
    """a = 12 where U >= 0, 3 elsewhere (Darcy_Gen.m:35-37)."""
    return np.where(U >= 0, 12.0, 3.0)


def centres(K: int) -> np.ndarray:
    return (2.0 * np.arange(K) + 1.0) / (2.0 * K)          # 1/(2K) : 1/K : (2K-1)/(2K)   (Solve_GWF.m:6)


def nodes(K: int) -> np.ndarray:
    return np.arange(K) / (K - 1.0)                        # 0 : 1/(K-1) : 1               (Solve_GWF.m:7)


def spline_resample(Z: np.ndarray, src: np.ndarray, dst: np.ndarray) -> np.ndarray:
    """Tensor-product not-a-knot cubic spline through Z on src x src, evaluated on dst x dst (interp2 'spline',
    Solve_GWF.m:9-10,41); points outside the source range are extrapolated by the end polynomials, as MATLAB does."""
    from scipy.interpolate import CubicSpline
    Z = CubicSpline(src, Z, axis=0, bc_type='not-a-knot', extrapolate=True)(dst)
    return CubicSpline(src, Z, axis=1, bc_type='not-a-knot', extrapolate=True)(dst)


def assemble(coef: np.ndarray):
    """The (K-2)^2 x (K-2)^2 matrix of Solve_GWF.m:16-35 for node coefficients coef [K, K], unknown (i, j) at
    index (i-1) * (K-2) + (j-1) (any consistent ordering gives the same solution):
        sum over the four neighbours n of (coef[n] + coef[i,j]) / 2 * (p[i,j] - p[n]) * (K-1)^2 = f[i,j]."""
    import scipy.sparse as sp
    K = coef.shape[0]
    n = K - 2
    c = coef[1:-1, 1:-1]
    wN = (coef[:-2, 1:-1] + c) / 2
    wS = (coef[2:, 1:-1] + c) / 2
    wW = (coef[1:-1, :-2] + c) / 2
    wE = (coef[1:-1, 2:] + c) / 2
    idx = np.arange(n * n).reshape(n, n)
    rows, cols, vals = [idx.ravel()], [idx.ravel()], [(wN + wS + wW + wE).ravel()]
    rows.append(idx[1:, :].ravel()); cols.append(idx[:-1, :].ravel()); vals.append(-wN[1:, :].ravel())
    rows.append(idx[:-1, :].ravel()); cols.append(idx[1:, :].ravel()); vals.append(-wS[:-1, :].ravel())
    rows.append(idx[:, 1:].ravel()); cols.append(idx[:, :-1].ravel()); vals.append(-wW[:, 1:].ravel())
    rows.append(idx[:, :-1].ravel()); cols.append(idx[:, 1:].ravel()); vals.append(-wE[:, :-1].ravel())
    A = sp.csr_matrix((np.concatenate(vals), (np.concatenate(rows), np.concatenate(cols))), shape=(n * n, n * n))
    return A * float((K - 1) ** 2)


def solve_nodes(coef_nodes: np.ndarray, f_nodes: np.ndarray) -> np.ndarray:
    """p on the K x K node grid, zero on the boundary (Solve_GWF.m:12,35,38)."""
    import scipy.sparse.linalg as spla
    K = coef_nodes.shape[0]
    A = assemble(coef_nodes).tocsc()
    x = spla.spsolve(A, f_nodes[1:-1, 1:-1].ravel())
    P = np.zeros((K, K))
    P[1:-1, 1:-1] = x.reshape(K - 2, K - 2)
    return P


def solve_gwf(coef: np.ndarray, F: np.ndarray) -> np.ndarray:
    """Solve_GWF.m: cell-centre fields in, cell-centre solution out.  (The original stores the interior solution
    transposed, resamples and transposes back; both grids are the same in x and y, so that is the identity.)"""
    K = coef.shape[0]
    cn = spline_resample(coef, centres(K), nodes(K))
    fn = spline_resample(F, centres(K), nodes(K))
    return spline_resample(solve_nodes(cn, fn), nodes(K), centres(K))


def darcy_gen(S: int, rng: np.random.Generator):
    """One (a, u) pair (Darcy_Gen.m:13-49): thresholded GRF(alpha 2, tau 3) and the solution for f = 1."""
    a = threshold_coefficient(gaussian_random_field(S, rng, 2.0, 3.0))
    return a, solve_gwf(a, np.ones((S, S)))


def poisson_unit_square(x: float, y: float, terms: int = 200) -> float:
    """Series solution of -laplace(p) = 1 on the unit square with p = 0 on the boundary."""
    s = 0.0
    for m in range(1, terms, 2):
        for n in range(1, terms, 2):
            s += 16.0 / (np.pi ** 4 * m * n * (m * m + n * n)) * np.sin(m * np.pi * x) * np.sin(n * np.pi * y)
    return s
