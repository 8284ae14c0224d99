"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (C0..C4).  They stand in for the translation /
pre-training batches the reference trains on; no dataset is needed.

Everything is drawn from one ``torch.Generator`` per configuration (seed
``20221 + config index``) on the CPU in fp32 and then cast/moved, so every rank
and every device count sees the same data; a rank takes a contiguous slice.

Conventions (fs_plugins/custom_ops/dag_loss.py:71-100):
  match_all [B,T,L]  log P(y_t | v_j)
  links     [B,L,K]  band format, links[b,i,d] = log P(v_i -> v_{i+d+1}), K = L-1
  output_length / target_length [B] int64
"""
import math
from dataclasses import dataclass
from typing import Optional

import torch

NEG_INF = float("-inf")
BASE_SEED = 20221
PAD_TOKEN = 1


def generator(config_index: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(BASE_SEED + int(config_index))
    return g


def square_to_band(sq: torch.Tensor, translen: Optional[int] = None) -> torch.Tensor:
    """square[b,i,j] -> band[b,i,j-i-1], -inf past the end
    (extract_valid_links, fs_plugins/models/glat_decomposed_with_link.py:319-335)."""
    B, L, _ = sq.shape
    K = L - 1 if translen is None else min(translen, L - 1)
    K = max(K, 1)
    idx = torch.arange(L, device=sq.device).unsqueeze(1) + torch.arange(K, device=sq.device).unsqueeze(0) + 1
    bad = idx >= L
    band = sq.gather(2, idx.clamp(max=L - 1).unsqueeze(0).expand(B, -1, -1))
    return band.masked_fill(bad.unsqueeze(0), NEG_INF).contiguous()


def band_to_square(band: torch.Tensor) -> torch.Tensor:
    """band[b,i,d] -> square[b,i,i+d+1], -inf elsewhere
    (restore_valid_links, fs_plugins/models/glat_decomposed_with_link.py:337-349)."""
    B, L, K = band.shape
    idx = torch.arange(L, device=band.device).unsqueeze(1) + torch.arange(K, device=band.device).unsqueeze(0) + 1
    idx = idx.masked_fill(idx >= L, L)
    res = torch.full((B, L, L + 1), NEG_INF, dtype=band.dtype, device=band.device)
    res.scatter_(2, idx.unsqueeze(0).expand(B, -1, -1), band)
    return res[:, :, :L].contiguous()


def make_links(B: int, L: int, output_length: torch.Tensor, gen: torch.Generator,
               translen: Optional[int] = None, chunk: int = 64, score_scale: float = 1.0) -> torch.Tensor:
    """Band links [B,L,K] fp32: row-wise log_softmax of N(0,1) scores over the valid
    successors (j > i, both below output_length); rows without a successor are all
    -inf (a bare log_softmax would give NaN there; the model writes -inf too,
    glat_decomposed_with_link.py:401-403)."""
    out = []
    ar = torch.arange(L)
    for s in range(0, B, chunk):
        e = min(B, s + chunk)
        ol = output_length[s:e].view(-1, 1, 1)
        scores = torch.randn(e - s, L, L, generator=gen, dtype=torch.float32)
        if score_scale != 1.0:
            scores = scores * score_scale
        valid = (ar.view(1, 1, L) > ar.view(1, L, 1)) & (ar.view(1, 1, L) < ol) & (ar.view(1, L, 1) < ol)
        scores = scores.masked_fill(~valid, NEG_INF)
        has = valid.any(-1, keepdim=True)
        sq = torch.log_softmax(scores.masked_fill(~has, 0.0), dim=-1).masked_fill(~valid, NEG_INF)
        out.append(square_to_band(sq, translen))
    return torch.cat(out, 0)


@dataclass
class DagBatch:
    """One batch of the hot path.  ``logits`` may be None when only the DP ops are
    exercised (``match_all`` is then given directly)."""
    name: str
    logits: Optional[torch.Tensor]        # [B,L,V]
    targets: torch.Tensor                 # [B,T] int64 (PAD_TOKEN at t >= target_length)
    links: torch.Tensor                   # [B,L,K] fp32 band
    output_length: torch.Tensor           # [B] int64
    target_length: torch.Tensor           # [B] int64
    match_all: Optional[torch.Tensor] = None  # [B,T,L] fp32

    @property
    def select_idx(self) -> torch.Tensor:
        """The stride-(T,0,1) expand the criterion passes
        (fs_plugins/criterions/nat_dag_loss.py:168)."""
        L = self.links.shape[1]
        return self.targets.unsqueeze(1).expand(-1, L, -1)

    def to(self, device):
        mv = lambda x: None if x is None else x.to(device)
        return DagBatch(self.name, mv(self.logits), mv(self.targets), mv(self.links),
                        mv(self.output_length), mv(self.target_length), mv(self.match_all))

    def shard(self, rank: int, world: int) -> "DagBatch":
        """Contiguous slice of the global batch for one rank."""
        B = self.targets.shape[0]
        per = (B + world - 1) // world
        s, e = rank * per, min(B, (rank + 1) * per)
        sl = lambda x: None if x is None else x[s:e]
        return DagBatch(self.name, sl(self.logits), sl(self.targets), sl(self.links),
                        sl(self.output_length), sl(self.target_length), sl(self.match_all))


def _targets(B, T, tl, V, gen, low=4):
    tok = torch.randint(low, V, (B, T), generator=gen, dtype=torch.int64)
    pad = torch.arange(T).view(1, T) >= tl.view(B, 1)
    return tok.masked_fill(pad, PAD_TOKEN)


def torch_match_from_logits(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """match_all [B,T,L] from logits [B,L,V] by plain torch ops (used to prepare
    inputs only): log_softmax in fp32, gather at the targets, transpose."""
    lp = torch.log_softmax(logits.float(), dim=-1)
    L = logits.shape[1]
    return lp.gather(-1, targets.unsqueeze(1).expand(-1, L, -1)).transpose(1, 2).contiguous()


def synthetic_match(B, T, L, V, sigma, gen) -> torch.Tensor:
    """match_all with the distribution a log-softmax over V iid N(0,sigma) logits
    gives at a random token: x - logsumexp, x ~ N(0,sigma), logsumexp concentrated at
    log V + sigma^2/2.  Used where materialising [B,L,V] logits is too large."""
    lse = math.log(V) + 0.5 * sigma * sigma
    return torch.randn(B, T, L, generator=gen, dtype=torch.float32) * sigma - lse


def config0(gen=None) -> DagBatch:
    """C0: B=8, L=160 (= output_length), target_length ~ U{10..20}, T=20, V=1000,
    fp32 logits N(0,1), tokens U{4..999}."""
    gen = gen or generator(0)
    B, L, T, V = 8, 160, 20, 1000
    tl = torch.randint(10, 21, (B,), generator=gen, dtype=torch.int64)
    T = int(tl.max())
    ol = torch.full((B,), L, dtype=torch.int64)
    logits = torch.randn(B, L, V, generator=gen, dtype=torch.float32)
    targets = _targets(B, T, tl, V, gen)
    links = make_links(B, L, ol, gen)
    return DagBatch("C0", logits, targets, links, ol, tl)


def config1(gen=None, B=64, V=42000, dtype=torch.float16, with_logits=True) -> DagBatch:
    """C1: B=64, source length ~ U{10..64}, output_length = 8*source, L = max (<=512),
    target_length = clip(round(U[0.8,1.2]*source), 2, 64), T = max, V=42000,
    fp16 logits N(0,2), fp32 links."""
    gen = gen or generator(1)
    src = torch.randint(10, 65, (B,), generator=gen, dtype=torch.int64)
    ol = 8 * src
    L = int(ol.max())
    ratio = torch.rand(B, generator=gen) * 0.4 + 0.8
    tl = torch.clamp(torch.round(ratio * src).to(torch.int64), 2, 64)
    T = int(tl.max())
    targets = _targets(B, T, tl, V, gen)
    links = make_links(B, L, ol, gen)
    logits = None
    match = None
    if with_logits:
        logits = (torch.randn(B, L, V, generator=gen, dtype=torch.float32) * 2.0).to(dtype)
    else:
        match = synthetic_match(B, T, L, V, 2.0, gen)
    return DagBatch("C1", logits, targets, links, ol, tl, match)


def config2(V=32000, dtype=torch.bfloat16, B=32, L=1024, S=128, gen=None):
    """C2: logsoftmax_gather sweep.  logits [B,L,V] N(0,2) in bf16/fp16,
    select_idx [B,L,S] int64 uniform over [0,V), contiguous."""
    gen = gen or generator(2)
    idx = torch.randint(0, V, (B, L, S), generator=gen, dtype=torch.int64)
    logits = torch.empty(B, L, V, dtype=dtype)
    for b in range(B):  # chunked so the fp32 staging copy stays small
        logits[b] = (torch.randn(L, V, generator=gen, dtype=torch.float32) * 2.0).to(dtype)
    return logits, idx


def config3(gen=None, B=16, L=1024, V=30522) -> DagBatch:
    """C3: B=16, L=1024, target_length ~ U{128..256}, T=256,
    output_length ~ U{4*tl..1024}, fp32 match/links, logits N(0,1) (represented by
    ``synthetic_match``: [16,1024,30522] fp32 logits are 2 GB)."""
    gen = gen or generator(3)
    tl = torch.randint(128, 257, (B,), generator=gen, dtype=torch.int64)
    T = int(tl.max())
    u = torch.rand(B, generator=gen)
    ol = (4 * tl + torch.floor(u * (L - 4 * tl + 1)).to(torch.int64)).clamp(max=L)
    targets = _targets(B, T, tl, V, gen)
    links = make_links(B, L, ol, gen, chunk=4)
    match = synthetic_match(B, T, L, V, 1.0, gen)
    return DagBatch("C3", None, targets, links, ol, tl, match)


def config4(gen=None, B=512, L=512, V=42000, tl_lo=32, tl_hi=64) -> DagBatch:
    """C4: global batch of 512 sentences, L=512 (= output_length), target_length ~
    U{32..64}, T=64, V=42000, bf16 logits N(0,2) (represented by ``synthetic_match``:
    the [512,512,42000] bf16 logits are 22 GB), fp32 links."""
    gen = gen or generator(4)
    tl = torch.randint(tl_lo, tl_hi + 1, (B,), generator=gen, dtype=torch.int64)
    T = tl_hi
    ol = torch.full((B,), L, dtype=torch.int64)
    targets = _targets(B, T, tl, V, gen)
    links = make_links(B, L, ol, gen)
    match = synthetic_match(B, T, L, V, 2.0, gen)
    return DagBatch("C4", None, targets, links, ol, tl, match)


def config4_peaky(gen=None, B=512, L=512, V=42000, tl_lo=32, tl_hi=64, score_scale=8.0) -> DagBatch:
    """C4 shapes with the value distribution of a TRAINED graph instead of a random one: transition
    scores N(0, score_scale) before the row softmax (a few successors carry almost all the mass), and
    match rows in which one vertex per target token is near probability one (log-prob -0.2) while
    the others sit near -15 +- 3 nats.  The dominant vertices increase with the target step and
    start / end on the first / last vertex, so every sentence keeps a likely path."""
    gen = gen or generator(40)
    tl = torch.randint(tl_lo, tl_hi + 1, (B,), generator=gen, dtype=torch.int64)
    T = tl_hi
    ol = torch.full((B,), L, dtype=torch.int64)
    targets = _targets(B, T, tl, V, gen)
    links = make_links(B, L, ol, gen, score_scale=score_scale)
    match = torch.randn(B, T, L, generator=gen, dtype=torch.float32) * 3.0 - 15.0
    for b in range(B):
        n = int(tl[b])
        inner = torch.sort(torch.randperm(L - 2, generator=gen)[: n - 2] + 1).values
        pos = torch.cat([torch.zeros(1, dtype=torch.long), inner, torch.full((1,), L - 1, dtype=torch.long)])
        match[b, torch.arange(n), pos] = -0.2
    return DagBatch("C4-peaky", None, targets, links, ol, tl, match)


def small_batch(seed=0, B=4, L=24, T=6, V=50, translen=None, ragged=True,
                dtype=torch.float32) -> DagBatch:
    """Tiny ragged batch for parity tests (sizes the CPU oracle finishes instantly)."""
    gen = torch.Generator(device="cpu")
    gen.manual_seed(1000 + seed)
    if ragged:
        tl = torch.randint(2, T + 1, (B,), generator=gen, dtype=torch.int64)
        tl[0] = T
        ol = torch.stack([torch.randint(int(t), L + 1, (1,), generator=gen)[0] for t in tl]).to(torch.int64)
        ol[0] = L
    else:
        tl = torch.full((B,), T, dtype=torch.int64)
        ol = torch.full((B,), L, dtype=torch.int64)
    logits = torch.randn(B, L, V, generator=gen, dtype=torch.float32).to(dtype)
    targets = _targets(B, T, tl, V, gen, low=min(4, V - 1))
    links = make_links(B, L, ol, gen, translen=translen)
    match = torch_match_from_logits(logits, targets)
    return DagBatch("small", logits, targets, links, ol, tl, match)
