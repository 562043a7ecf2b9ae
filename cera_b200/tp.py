"""Tensor-parallel plumbing above the C ABI: which rows of which tensor a rank keeps, and the
exchange of the ranks' region handles through torch.distributed (one process per GPU).

The split is by output rows of the feed-forward matrices and the LM head, the one axis cera parallelises on the CPU
(cera/src/backend/cpu.rs:380-391): a row's dot product is the same arithmetic on any number of
ranks, so a tensor-parallel model reproduces the single-GPU logits.  The device side of the
exchange is csrc/tp.cu."""
from .model import Role

#: roles whose rows are split: the feed-forward matrices (four fifths of a layer's bytes) and the LM head.  Everything else
#: is replicated - norm vectors, embedding table, rope factors, and the whole attention block (q / k / v, KV cache, o-proj):
#: its launches are latency-bound whole or split, and a rank that holds all heads needs no exchange around the attention
SPLIT_ROLES = (Role.FFN_GATE, Role.FFN_UP, Role.FFN_DOWN, Role.OUTPUT)


def check_divisible(cfg, size):
    """Same rules as cera_cuda_model_set_tp; raises ValueError naming the first one broken."""
    if not 1 <= size <= 8:
        raise ValueError(f"tensor parallel size {size} outside 1..8")
    if cfg.n_kv_heads % size:
        raise ValueError(f"{cfg.n_kv_heads} KV heads do not split over {size} ranks")
    if cfg.intermediate_size % (32 * size):
        raise ValueError(f"intermediate size {cfg.intermediate_size} is not a multiple of 32 x {size}")
    if cfg.hidden_size % size or cfg.vocab_size % size:
        raise ValueError(f"hidden size {cfg.hidden_size} / vocabulary {cfg.vocab_size} not divisible by {size}")


def row_range(role, rows, rank, size):
    """[first, last) rows of a tensor with `rows` rows that rank `rank` of `size` keeps."""
    if Role(role) not in SPLIT_ROLES or size == 1:
        return 0, rows
    if rows % size:
        raise ValueError(f"{rows} rows of {Role(role).name} do not split over {size} ranks")
    per = rows // size
    return rank * per, (rank + 1) * per


def exchange_slots(n_layers):
    """Exchange slots of one decode step: four per layer (two unused since the attention block is whole on every rank,
    SwiGLU activations, residual after the down-proj), then the logits slice or the greedy pair."""
    return 4 * n_layers + 1


def gather_handles(handle, group=None):
    """All ranks' 64-byte region handles in rank order (works on any backend: gloo on CPU, nccl on GPUs)."""
    import torch.distributed as dist
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, bytes(handle), group=group)
    if any(len(h) != len(handle) for h in out):
        raise RuntimeError("ranks disagree on the handle size")
    return out


def connect(model, group=None):
    """Finalized tensor-parallel model -> connected to its peers.  Collective: every rank calls it."""
    import torch.distributed as dist
    rank, size = model.tp
    if size == 1:
        return
    if dist.get_world_size(group) != size or dist.get_rank(group) != rank:
        raise RuntimeError(f"model is rank {rank} of {size} but the process group says "
                           f"{dist.get_rank(group)} of {dist.get_world_size(group)}")
    model.tp_connect(gather_handles(model.tp_handle(), group))
    dist.barrier(group)
