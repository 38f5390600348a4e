"""Greedy decoding with the tensor-parallel language models (inference through the same layers and kernels).

The reference runs inference by handing its patched Hugging Face models to ``generate``; the models of this
package return logits whose vocabulary dimension is split over the ranks of ``model.head.group``, so choosing the
next token is a small collective: every rank proposes its best local candidate and all ranks pick the same winner.
"""

import torch
import torch.distributed as dist


@torch.no_grad()
def parallel_argmax(logits, group=None):
    """``argmax`` over a last dimension that is split over ``group`` in rank order (``None``: not split).  Every
    rank returns the same global indices; ties go to the lowest index, as in ``torch.argmax`` of the whole row."""
    value, index = logits.float().max(dim=-1)
    if group is None or dist.get_world_size(group) == 1:
        return index
    n, me = dist.get_world_size(group), dist.get_rank(group)
    index = index + me * logits.shape[-1]
    values = [torch.empty_like(value) for _ in range(n)]
    indices = [torch.empty_like(index) for _ in range(n)]
    dist.all_gather(values, value.contiguous(), group=group)
    dist.all_gather(indices, index.contiguous(), group=group)
    values, indices = torch.stack(values, -1), torch.stack(indices, -1)      # [..., n]; rank order = index order
    best = values.argmax(dim=-1, keepdim=True)                               # first maximum = lowest rank
    return indices.gather(-1, best).squeeze(-1)


@torch.no_grad()
def greedy_generate(model, tokens, max_new_tokens: int, eos_id=None):
    """Extend ``tokens`` ``[B, S0]`` by up to ``max_new_tokens`` greedily chosen tokens; returns ``[B, S0 + new]``.

    Every rank of a tensor-parallel group passes the same ``tokens`` (ranks that differ in data or depth
    coordinates may pass different batches).  The whole prefix is re-evaluated for every new token (no key/value
    cache), which keeps the attention kernels' training-time code path; sequences stop growing for rows that have
    produced ``eos_id``, which are padded with it.  The model is left in evaluation mode for the call."""
    was_training = model.training
    model.eval()
    limit = getattr(getattr(model, "cfg", None), "seq_len", None)
    done = torch.zeros(tokens.shape[0], dtype=torch.bool, device=tokens.device)
    try:
        for _ in range(max_new_tokens):
            if limit is not None and tokens.shape[1] >= limit:
                break
            logits = model(tokens)                                           # [B, S, vocab / |group|]
            nxt = parallel_argmax(logits[:, -1], getattr(model.head, "group", None)).to(tokens.dtype)
            if eos_id is not None:
                nxt = torch.where(done, torch.full_like(nxt, eos_id), nxt)
                done = done | (nxt == eos_id)
            tokens = torch.cat([tokens, nxt[:, None]], dim=1)
            if eos_id is not None and bool(done.all()):
                break
    finally:
        model.train(was_training)
    return tokens
