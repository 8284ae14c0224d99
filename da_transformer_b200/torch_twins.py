"""PyTorch-native twins of the three ops, with the names and conventions of the reference's
`torch_dag_loss`, `torch_dag_best_alignment`, `torch_dag_logsoftmax_gather_inplace`
(fs_plugins/custom_ops/dag_loss.py:259-359), so that `fs_plugins/custom_ops/__init__.py` can
take all six names from this package.  They are what the criterion's `--torch-dag-loss`,
`--torch-dag-best-alignment`, `--torch-dag-logsoftmax-gather` flags select
(fs_plugins/criterions/nat_dag_loss.py:59-64) and what the model's graph analysis calls
(fs_plugins/models/glat_decomposed_with_link.py:572-575).

Plain differentiable torch code for any device.  They are NOT a fallback of the CUDA ops:
`dag_loss`, `dag_best_alignment` and `dag_logsoftmax_gather_inplace` never route here.

NOTE the reference's convention: these take SQUARE links [B, L, L] (links[b,i,j] = transition
i -> j, -inf for j <= i), not the band format of the CUDA ops.
"""
import torch

NEG_INF = float("-inf")


def _logsumexp_over_predecessors(x: torch.Tensor) -> torch.Tensor:
    """log sum_i exp(x[b,i,j]) over dim 1, exact -inf (and zero gradient) where every term is -inf."""
    m = x.max(dim=1, keepdim=True).values
    dead = m == NEG_INF
    shift = torch.where(dead, torch.zeros_like(m), m).detach()
    s = (x - shift).exp().sum(dim=1, keepdim=True)
    out = torch.where(dead, torch.ones_like(s), s).log() + shift
    return torch.where(dead, torch.full_like(out, NEG_INF), out).squeeze(1)


def _forward_rows(match_all, links, reduce_fn):
    bsz, tarlen, prelen = match_all.shape
    if links.dim() != 3 or links.shape[1] != links.shape[2] or links.shape[1] != prelen:
        raise AssertionError("links should be batch_size * prelen * prelen")
    first = torch.full((bsz, prelen), NEG_INF, dtype=match_all.dtype, device=match_all.device)
    first = torch.cat([match_all[:, 0, :1], first[:, 1:]], dim=1)
    rows = [first]
    for t in range(1, tarlen):
        rows.append(reduce_fn(rows[-1].unsqueeze(2) + links) + match_all[:, t])
    return torch.stack(rows, dim=1)  # [B, T, L]


def torch_dag_loss(match_all, links, output_length, target_length):
    """log P(target | graph) per sentence; match_all [B,T,L], links [B,L,L] square."""
    rows = _forward_rows(match_all, links, _logsumexp_over_predecessors)
    b = torch.arange(match_all.shape[0], device=match_all.device)
    return rows[b, target_length - 1, output_length - 1]


def torch_dag_best_alignment(match_all, links, output_length, target_length):
    """Best alignment by explicit Viterbi + backtrace; returns [B,L] int64, -1 = not aligned.
    Among exactly equal candidates the first (smallest) predecessor wins, which differs from the
    CUDA op's tie-break; on tie-free inputs the two agree."""
    with torch.no_grad():
        bsz, tarlen, prelen = match_all.shape
        score = torch.full((bsz, prelen), NEG_INF, dtype=match_all.dtype, device=match_all.device)
        score[:, 0] = match_all[:, 0, 0]
        back = []
        for t in range(1, tarlen):
            best, arg = (score.unsqueeze(2) + links).max(dim=1)
            back.append(arg)
            score = best + match_all[:, t]
        path = torch.full((bsz, prelen), -1, dtype=torch.long, device=match_all.device)
        b = torch.arange(bsz, device=match_all.device)
        pos = (output_length - 1).clone()
        for t in range(tarlen - 1, -1, -1):
            active = t <= (target_length - 1)
            pos = torch.where(t == target_length - 1, output_length - 1, pos)
            current = path[b, pos]
            path[b, pos] = torch.where(active, torch.full_like(current, t), current)
            if t > 0:
                pos = torch.where(active, back[t - 1][b, pos], pos)
        return path


def torch_dag_logsoftmax_gather_inplace(word_ins_out, select_idx):
    """(word_ins_out, log_softmax(word_ins_out, fp32).gather(-1, select_idx)); not in place."""
    logp = torch.log_softmax(word_ins_out, dim=-1, dtype=torch.float32)
    return word_ins_out, logp.gather(dim=-1, index=select_idx)
