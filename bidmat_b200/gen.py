"""Seeded synthetic inputs with the shapes and distributions of the five
benchmark configurations of the sparse-dense path.  They stand in for real
LDA / factorisation data; nothing here reads a dataset.

Everything is produced with torch on the requested device (CPU or CUDA) from a
torch.Generator seeded by the caller, so a (config, scale, seed, device type)
tuple always gives the same matrices.  `scale` shrinks the matrix dimensions
(and the column-length clip) proportionally; scale=1 is the full size.

Structure rules kept so that "same structure" is unambiguous
(src/main/scala/BIDMat/SparseMat.scala:710-740, 671-708): rows strictly
increasing inside a column, jc[0] = 0, jc[n] = nnz, no stored zeros.

Dense operands are returned as (ncols, k) tensors = column-major k x ncols.
"""
import math
from dataclasses import dataclass

import torch


@dataclass
class Problem:
    name: str
    k: int
    m: int          # rows of S
    n: int          # columns of S
    jc: torch.Tensor    # int32 (n+1)
    ir: torch.Tensor    # int32 (nnz)
    data: torch.Tensor  # float32 (nnz)
    A: torch.Tensor     # float32 (m, k) or None
    B: torch.Tensor     # float32 (n, k) or None

    @property
    def nnz(self):
        return int(self.ir.numel())


def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def _nonzero_uniform(nnz, g, device):
    v = torch.rand(nnz, generator=g, device=device, dtype=torch.float32)
    return torch.clamp_min(v, 2.0 ** -24)   # U(0,1) draws that round to 0 would be stripped as stored zeros


def _csc_from_keys(keys, m, n):
    """keys = col*m + row, sorted and unique -> (jc, ir)."""
    cols = torch.div(keys, m, rounding_mode="floor")
    ir = (keys - cols * m).to(torch.int32)
    counts = torch.bincount(cols, minlength=n)
    jc = torch.zeros(n + 1, dtype=torch.int64, device=keys.device)
    torch.cumsum(counts, 0, out=jc[1:])
    return jc.to(torch.int32), ir


def fixed_length_columns(m, n, per_col, g, device):
    """Exactly `per_col` distinct rows per column, uniform without replacement,
    sorted.  Over-draw with replacement, drop duplicates, then keep a random
    subset of the right size in every column (a random subset of a uniform
    distinct sample is again uniform)."""
    per_col = min(per_col, m)
    over = per_col + max(8, int(0.25 * per_col))
    while True:
        rows = torch.randint(0, m, (n, over), generator=g, device=device, dtype=torch.int64)
        keys = (torch.arange(n, device=device, dtype=torch.int64).unsqueeze(1) * m + rows).flatten()
        keys = torch.unique(keys)      # sorted
        cols = torch.div(keys, m, rounding_mode="floor")
        counts = torch.bincount(cols, minlength=n)
        if int(counts.min()) >= per_col:
            break
        over = min(2 * over, max(m, over + 1)) if over < m else over * 2
    # random priority per entry; keep the per_col smallest priorities of each column
    pri = torch.rand(keys.numel(), generator=g, device=device, dtype=torch.float64)
    order = torch.argsort(cols.to(torch.float64) + pri * 0.999999)   # by column, then priority
    start = torch.zeros(n + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=start[1:])
    rank = torch.arange(keys.numel(), device=device) - start[cols[order]]
    keep = order[rank < per_col]
    keys = torch.sort(keys[keep]).values
    return _csc_from_keys(keys, m, n)


def zipf_cdf(m, s, device):
    w = torch.arange(1, m + 1, device=device, dtype=torch.float64).pow(-s)
    cdf = torch.cumsum(w, 0)
    return (cdf / cdf[-1]).to(torch.float64)


def zipf_columns(m, n, lengths, s, g, device, block=1 << 26):
    """Column c gets `lengths[c]` Zipf(s) draws over [0, m) (row 0 the most
    frequent), de-duplicated and sorted; realised lengths are <= drawn ones.
    Draws are processed in blocks of columns to bound memory."""
    cdf = zipf_cdf(m, s, device)
    lengths = lengths.to(torch.int64)
    csum = torch.cumsum(lengths, 0)
    total = int(csum[-1])
    keys_out = []
    c0 = 0
    while c0 < n:
        # largest c1 with draws(c0..c1) <= block (at least one column)
        base = int(csum[c0 - 1]) if c0 > 0 else 0
        c1 = int(torch.searchsorted(csum, torch.tensor([base + block], device=device), right=True))
        c1 = max(c1, c0 + 1)
        c1 = min(c1, n)
        lens = lengths[c0:c1]
        cnt = int(lens.sum())
        cols = torch.repeat_interleave(torch.arange(c0, c1, device=device, dtype=torch.int64), lens)
        u = torch.rand(cnt, generator=g, device=device, dtype=torch.float64)
        rows = torch.searchsorted(cdf, u).clamp_(max=m - 1)
        keys_out.append(torch.unique(cols * m + rows))
        del cols, u, rows
        c0 = c1
    keys = torch.cat(keys_out) if len(keys_out) > 1 else keys_out[0]
    del keys_out
    assert total >= keys.numel()
    return _csc_from_keys(keys, m, n)


def _normal(shape, g, device, std=1.0):
    out = torch.empty(shape, dtype=torch.float32, device=device)
    out.normal_(0.0, std, generator=g)
    return out


def config1(scale=1.0, seed=0, device="cpu"):
    """CPU-runnable baseline: k=128, S 100000 x 20000 with exactly 100 nnz per
    column (uniform rows without replacement, sorted), values U(0,1);
    A 128 x 100000 and B 128 x 20000 N(0,1)."""
    g = _gen(device, seed)
    k = 128
    m = max(128, int(round(100_000 * scale)))
    n = max(16, int(round(20_000 * scale)))
    jc, ir = fixed_length_columns(m, n, 100, g, device)
    data = _nonzero_uniform(ir.numel(), g, device)
    return Problem("config1", k, m, n, jc, ir, data, _normal((m, k), g, device), _normal((n, k), g, device))


def lda_structure(m, n, g, device, mu=5.0, sigma=0.8, clip=20_000, zipf_s=1.1):
    lengths = torch.empty(n, dtype=torch.float64, device=device).normal_(mu, sigma, generator=g).exp_()
    lengths = lengths.round().clamp_(1, max(1, clip)).to(torch.int64)
    return zipf_columns(m, n, lengths, zipf_s, g, device)


def config2(scale=1.0, seed=0, device="cpu", with_A=True, with_B=True):
    """LDA-shaped counts: S 1e6 x 1e6, column lengths log-normal(5.0, 0.8)
    clipped to [1, 20000], rows Zipf(1.1) de-duplicated and sorted, values
    1+Poisson(0.5); A 256 x 1e6 U(0, 1/256); B 256 x 1e6 N(0,1).  Config 4 (the
    transposed-product model update) uses the same S and B."""
    g = _gen(device, seed)
    k = 256
    m = max(256, int(round(1_000_000 * scale)))
    n = max(16, int(round(1_000_000 * scale)))
    jc, ir = lda_structure(m, n, g, device, clip=max(8, int(round(20_000 * min(1.0, scale * 4)))))
    lam = torch.full((ir.numel(),), 0.5, dtype=torch.float32, device=device)
    data = 1.0 + torch.poisson(lam, generator=g)
    del lam
    A = torch.rand((m, k), generator=g, device=device, dtype=torch.float32).mul_(1.0 / 256) if with_A else None
    B = _normal((n, k), g, device) if with_B else None
    return Problem("config2", k, m, n, jc, ir, data, A, B)


def config3(k, scale=1.0, seed=0, device="cpu"):
    """SDDMM width sweep: S 500000 x 500000 with 64 uniform sorted rows per
    column, values U(0,1); A and B k x 500000 N(0,1); k in {32,...,512}."""
    g = _gen(device, seed)
    m = n = max(64, int(round(500_000 * scale)))
    jc, ir = fixed_length_columns(m, n, 64, g, device)
    data = _nonzero_uniform(ir.numel(), g, device)
    return Problem("config3_k%d" % k, k, m, n, jc, ir, data, _normal((m, k), g, device), _normal((n, k), g, device))


def config5(scale=1.0, seed=0, device="cpu", with_dense=True):
    """Skewed factorisation step: S 2e6 x 4e6, rows Zipf(1.05), column lengths
    Pareto(alpha=1.2, minimum 10) clipped at 200000, values U(0,1);
    A 128 x 2e6 and B 128 x 4e6 N(0, 0.1)."""
    g = _gen(device, seed)
    k = 128
    m = max(128, int(round(2_000_000 * scale)))
    n = max(16, int(round(4_000_000 * scale)))
    u = torch.rand(n, generator=g, device=device, dtype=torch.float64).clamp_min_(1e-12)
    lengths = (10.0 * u.pow(-1.0 / 1.2)).round().clamp_(10, max(10, int(round(200_000 * min(1.0, scale * 4)))))
    jc, ir = zipf_columns(m, n, lengths.to(torch.int64), 1.05, g, device)
    data = _nonzero_uniform(ir.numel(), g, device)
    A = _normal((m, k), g, device, std=0.1) if with_dense else None
    B = _normal((n, k), g, device, std=0.1) if with_dense else None
    return Problem("config5", k, m, n, jc, ir, data, A, B)


def sprand_like(m, n, density, seed=0, device="cpu"):
    """Small random CSC pattern in the spirit of BIDMat's sprand
    (src/main/scala/BIDMat/Random.scala:58-80): geometric gaps between
    successive nonzeros in column-major order, values U(0,1)."""
    g = _gen(device, seed)
    total = m * n
    cap = max(min(total, 200), int(1.5 * density * total))
    u = torch.rand(cap, generator=g, device=device, dtype=torch.float64).clamp_min_(1e-12)
    gaps = torch.floor(torch.log(u) / math.log(max(1e-12, 1.0 - density))).to(torch.int64)
    pos = torch.cumsum(gaps + 1, 0) - 1
    pos = pos[pos < total]
    keys = (pos % n) * m + torch.div(pos, n, rounding_mode="floor")   # any fixed bijection; then sort
    keys = torch.unique(keys)
    jc, ir = _csc_from_keys(keys, m, n)
    data = _nonzero_uniform(ir.numel(), g, device)
    return jc, ir, data


def shard_columns(jc, nshards):
    """Contiguous column ranges with (nearly) equal nonzero counts: returns
    nshards+1 column boundaries chosen by binary search in jc."""
    n = jc.numel() - 1
    nnz = int(jc[n])
    targets = torch.tensor([nnz * i // nshards for i in range(1, nshards)], dtype=jc.dtype, device=jc.device)
    cuts = torch.searchsorted(jc.contiguous(), targets).clamp_(0, n).tolist() if nshards > 1 else []
    bounds = [0] + [int(c) for c in cuts] + [n]
    for i in range(1, len(bounds)):
        bounds[i] = max(bounds[i], bounds[i - 1])
    return bounds
