"""
Tensor parallelism with sequence parallelism (the layouts of the reference's DTensor plans in
src/olmo_core/nn/attention/__init__.py:690-760, src/olmo_core/nn/feed_forward.py:172-204,
src/olmo_core/nn/transformer/block.py:231-262, src/olmo_core/nn/lm_head.py:300-370).

* Between sub-layers the activations are sharded along the *sequence*: ``[B, T/tp, D]`` per rank.
* Attention and MLP are column-parallel on the way in (``w_q/w_k/w_v`` by heads, ``w1/w3`` by hidden units) and
  row-parallel on the way out (``w_out``, ``w2``): the sequence shards are all-gathered in front of the first
  projections and the partial outputs are reduce-scattered back to sequence shards after the last one.
* Norms, embeddings and the LM head stay replicated. Parameters that only see a sequence shard (block norms) get partial
  gradients, which the sharded-parameter runtime sums over the tensor-parallel group (flag ``_tp_partial_grad``).

Parameters are sliced in place, so a tensor-parallel rank owns plain local tensors and every kernel-backed op works
unchanged on its slice. The collectives are autograd functions over the process group.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

__all__ = [
    "gather_from_sequence_parallel",
    "scatter_to_sequence_parallel",
    "all_gather_sequence",
    "reduce_scatter_sequence",
    "tp_full_width_rms_norm",
    "shard_attention_",
    "shard_feed_forward_",
    "shard_block_",
    "shard_lm_head_",
    "sum_partials",
    "local_sequence_shard",
    "shard_model_",
]


def _all_gather_seq(x: torch.Tensor, group) -> torch.Tensor:
    ws = dist.get_world_size(group)
    parts = [torch.empty_like(x) for _ in range(ws)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=1)


def _reduce_scatter_seq(x: torch.Tensor, group) -> torch.Tensor:
    ws = dist.get_world_size(group)
    chunks = [c.contiguous() for c in x.chunk(ws, dim=1)]
    out = torch.empty_like(chunks[0])
    if x.is_cuda:
        dist.reduce_scatter(out, chunks, op=dist.ReduceOp.SUM, group=group)
    else:  # gloo has no reduce-scatter
        full = x.contiguous()
        dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
        out = full.chunk(ws, dim=1)[dist.get_rank(group)].contiguous()
    return out


def _slice_seq(x: torch.Tensor, group) -> torch.Tensor:
    return x.chunk(dist.get_world_size(group), dim=1)[dist.get_rank(group)].contiguous()


class _GatherForPartialConsumer(torch.autograd.Function):
    """all-gather along the sequence; the consumer is column-parallel, so gradients are partial sums: reduce-scatter."""

    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        ctx.group = group
        return _all_gather_seq(x, group)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return _reduce_scatter_seq(g, ctx.group), None


class _ReduceScatterPartial(torch.autograd.Function):
    """reduce-scatter partial outputs of a row-parallel projection to sequence shards; backward all-gathers."""

    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        ctx.group = group
        return _reduce_scatter_seq(x, group)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return _all_gather_seq(g, ctx.group), None


class _GatherForReplicatedConsumer(torch.autograd.Function):
    """all-gather along the sequence; every rank then computes the same thing, so backward just takes the local slice."""

    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        ctx.group = group
        return _all_gather_seq(x, group)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return _slice_seq(g, ctx.group), None


class _ScatterFromReplicatedProducer(torch.autograd.Function):
    """take the local sequence slice of a replicated tensor; backward all-gathers (the producer needs the full gradient)."""

    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        ctx.group = group
        return _slice_seq(x, group)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return _all_gather_seq(g, ctx.group), None


class _ScatterKeepingLocalGradient(torch.autograd.Function):
    """take the local sequence slice of a replicated tensor; backward leaves the other ranks' positions at zero, so the
    producer's parameters receive this rank's part of their gradient only (a partial sum over the group)."""

    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        ctx.group = group
        ctx.seq = x.shape[1]
        return _slice_seq(x, group)

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        ws, rank = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        n = ctx.seq // ws
        full = g.new_zeros((g.shape[0], ctx.seq) + tuple(g.shape[2:]))
        full[:, rank * n:(rank + 1) * n] = g
        return full, None


def all_gather_sequence(x: torch.Tensor, group) -> torch.Tensor:
    """``[B, T/tp, ...] -> [B, T, ...]`` in front of a column-parallel projection."""
    return _GatherForPartialConsumer.apply(x, group)


def reduce_scatter_sequence(x: torch.Tensor, group) -> torch.Tensor:
    """Sum partial ``[B, T, ...]`` outputs over the group and keep this rank's ``[B, T/tp, ...]``."""
    return _ReduceScatterPartial.apply(x, group)


def gather_from_sequence_parallel(x: torch.Tensor, group) -> torch.Tensor:
    """``[B, T/tp, ...] -> [B, T, ...]`` for a consumer that every rank evaluates identically (the LM head)."""
    return _GatherForReplicatedConsumer.apply(x, group)


def scatter_to_sequence_parallel(x: torch.Tensor, group, partial_producer_grads: bool = False) -> torch.Tensor:
    """
    Local sequence shard of a tensor that every rank computed identically (the embeddings). By default the producer
    gets the whole gradient on every rank (all-gather in backward). With ``partial_producer_grads`` it gets this rank's
    part only: for producers whose parameters are summed over the group anyway (an embedding tied to the
    sequence-parallel head).
    """
    if partial_producer_grads:
        return _ScatterKeepingLocalGradient.apply(x, group)
    return _ScatterFromReplicatedProducer.apply(x, group)


class _SumPartialsForReplicatedConsumer(torch.autograd.Function):
    """Sum of per-rank partial results that every rank then uses identically (a loss summed over sequence shards): each
    rank's partial enters the total with weight one, so the gradient passes through unchanged."""

    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        y = x.clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        return y

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        return g, None


def sum_partials(x: torch.Tensor, group) -> torch.Tensor:
    """Total over the group of a quantity each rank computed for its own sequence shard."""
    return _SumPartialsForReplicatedConsumer.apply(x, group)


def local_sequence_shard(x: torch.Tensor, group) -> torch.Tensor:
    """This rank's ``[B, T/tp, ...]`` part of a tensor that needs no gradient (labels, masks)."""
    return _slice_seq(x, group)


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):  # type: ignore[override]
        ctx.group = group
        y = x.clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        return y

    @staticmethod
    def backward(ctx, g):  # type: ignore[override]
        g = g.clone()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


def tp_full_width_rms_norm(norm: nn.Module, t: torch.Tensor, group) -> torch.Tensor:
    """
    RMSNorm over a feature dimension that is split across the group (QK-norm over all heads with heads sharded): the
    mean of squares is formed from every rank's partial sum of squares, the (sliced) weight is applied locally.
    """
    ws = dist.get_world_size(group)
    x = t.float() if getattr(norm, "full_precision", True) else t
    local_sq = x.pow(2).sum(dim=-1, keepdim=True)
    total_sq = _AllReduceSum.apply(local_sq, group)
    width = t.shape[-1] * ws
    y = x * torch.rsqrt(total_sq / width + norm.eps)
    if getattr(norm, "weight", None) is not None:
        from ..ops.param import full_param

        w = full_param(norm.weight, y.dtype)
        y = y * w
    if getattr(norm, "bias", None) is not None:
        y = y + norm.bias.to(y.dtype)
    return y.to(t.dtype)


# ---------------------------------------------------------------------------------------------------------
# in-place sharding of parameters
# ---------------------------------------------------------------------------------------------------------
def _slice_param(module: nn.Module, name: str, dim: int, rank: int, ws: int, group=None) -> None:
    p = getattr(module, name, None)
    if p is None:
        return
    if p.shape[dim] % ws != 0:
        raise ValueError(f"cannot split dimension {dim} of '{name}' {tuple(p.shape)} over {ws} tensor-parallel ranks")
    n = p.shape[dim] // ws
    if p.device.type == "meta":
        shape = list(p.shape)
        shape[dim] = n
        new = torch.empty(shape, dtype=p.dtype, device="meta")
    else:
        new = p.data.narrow(dim, rank * n, n).clone()
    module._parameters[name] = nn.Parameter(new, requires_grad=p.requires_grad)
    module._parameters[name]._tp_sharded = True  # type: ignore[attr-defined]


def _column_parallel(linear: nn.Module, rank: int, ws: int) -> None:
    _slice_param(linear, "weight", 0, rank, ws)
    _slice_param(linear, "bias", 0, rank, ws)
    if hasattr(linear, "out_features"):
        linear.out_features //= ws


def _row_parallel(linear: nn.Module, rank: int, ws: int) -> None:
    _slice_param(linear, "weight", 1, rank, ws)
    if getattr(linear, "bias", None) is not None:
        # the bias is added on every rank before the reduce-scatter: keep 1/ws of it on each
        with torch.no_grad():
            if linear.bias.device.type != "meta":
                linear.bias.div_(ws)
    if hasattr(linear, "in_features"):
        linear.in_features //= ws


def _mark_partial(module: Optional[nn.Module], group) -> None:
    """Parameters of ``module`` see only a sequence shard: their gradients must be summed over ``group``."""
    if module is None:
        return
    for p in module.parameters():
        p._tp_partial_grad = group  # type: ignore[attr-defined]


def _mesh_info(tp_mesh):
    group = tp_mesh.get_group()
    return group, dist.get_rank(group), dist.get_world_size(group)


def _wrap_forward(module: nn.Module, group) -> None:
    """Gather the sequence shards in front of ``module`` and reduce-scatter its partial outputs."""
    if getattr(module, "_tp_wrapped", False):
        return
    inner = module.forward

    def forward(x, *args, **kwargs):
        return reduce_scatter_sequence(inner(all_gather_sequence(x, group), *args, **kwargs), group)

    module.forward = forward  # type: ignore[method-assign]
    module._tp_wrapped = True  # type: ignore[attr-defined]


def shard_attention_(attn: nn.Module, tp_mesh) -> None:
    """Split the heads over the group: ``w_q/w_k/w_v`` (and gates) column-parallel, ``w_out`` row-parallel."""
    group, rank, ws = _mesh_info(tp_mesh)
    if attn.n_heads % ws != 0 or attn.n_kv_heads % ws != 0:
        raise ValueError(f"{attn.n_heads} query / {attn.n_kv_heads} key-value heads do not divide over {ws} ranks")
    for name in ("w_q", "w_k", "w_v", "w_g"):
        if getattr(attn, name, None) is not None:
            _column_parallel(getattr(attn, name), rank, ws)
    _row_parallel(attn.w_out, rank, ws)
    for name in ("q_norm", "k_norm"):
        norm = getattr(attn, name, None)
        if norm is None:
            continue
        w = getattr(norm, "weight", None)
        if w is not None and w.numel() > attn.head_dim:  # a norm over all heads: its weight follows the head split
            _slice_param(norm, "weight", 0, rank, ws)
            _slice_param(norm, "bias", 0, rank, ws)
            norm._tp_full_width = True  # type: ignore[attr-defined]
        else:  # per-head norm: shared weight, partial gradients
            _mark_partial(norm, group)
    attn.n_heads //= ws
    attn.n_kv_heads //= ws
    if hasattr(attn, "backend"):
        for key in ("n_heads", "n_kv_heads"):
            if hasattr(attn.backend, key):
                setattr(attn.backend, key, getattr(attn, key))
    attn.tp_group = group
    inner = attn.forward
    _wrap_forward(attn, group)
    _fuse_attention(attn, group, inner)


def _fuse_attention(attn: nn.Module, group, inner) -> None:
    """
    Route the attention projections through the kernels that carry the collective themselves (as the MLP below): q, k
    and v gather the sequence shards of their input while they run, the output projection reduces its partial sums into
    the owners' shards. Falls back to the gather / reduce-scatter wrapper for biases, gates, KV caches, fp8 projections,
    CPU tensors, or when peer memory is unavailable.
    """
    from .tp_fused import fused_tp_available

    if not hasattr(attn, "_tp_project_in"):
        return
    wrapped = attn.forward
    projections = [getattr(attn, n, None) for n in ("w_q", "w_k", "w_v", "w_out")]
    if any(p is None or getattr(p, "bias", None) is not None for p in projections) or getattr(attn, "w_g", None) is not None:
        return

    def forward(x, *args, **kwargs):
        rows = x.numel() // x.shape[-1]
        if (getattr(attn, "kv_cache_manager", None) is not None or getattr(attn, "clip_qkv", None) is not None
                or any(getattr(p, "float8", None) is not None for p in projections)
                or not fused_tp_available(x, group, rows)):
            return wrapped(x, *args, **kwargs)
        attn._tp_fused_call = True
        try:
            return inner(x, *args, **kwargs)
        finally:
            attn._tp_fused_call = False

    attn.forward = forward  # type: ignore[method-assign]


def shard_feed_forward_(ff: nn.Module, tp_mesh) -> None:
    group, rank, ws = _mesh_info(tp_mesh)
    _column_parallel(ff.w1, rank, ws)
    _column_parallel(ff.w3, rank, ws)
    _row_parallel(ff.w2, rank, ws)
    if hasattr(ff, "hidden_size"):
        ff.hidden_size //= ws
    ff.tp_group = group  # type: ignore[attr-defined]
    _wrap_forward(ff, group)
    _fuse_feed_forward(ff, group)


def _fuse_feed_forward(ff: nn.Module, group) -> None:
    """
    Route a bias-free SwiGLU MLP through the kernels that carry the collective themselves: both up-projections gather
    their input from the peers while they run, the down-projection reduces its partial sums into the owners' shards from
    its epilogue. The MLP acts on rows independently, so the rank-major row order of the gathered activations needs no
    re-ordering. Anything else (biases, other activations, CPU tensors, no peer memory) keeps the wrapped forward.
    """
    from ..nn.feed_forward import ActivationFunction
    from ..ops.elementwise import swiglu
    from .tp_fused import fused_tp_available, gather_linear_multi, linear_reduce_scatter

    wrapped = ff.forward
    if (getattr(ff, "activation", None) != ActivationFunction.silu
            or any(getattr(getattr(ff, n), "bias", None) is not None for n in ("w1", "w2", "w3"))):
        return

    def forward(x, *args, **kwargs):
        rows = x.numel() // x.shape[-1]
        if (args or kwargs or not fused_tp_available(x, group, rows)
                or any(getattr(getattr(ff, n), "float8", None) is not None for n in ("w1", "w2", "w3"))):
            return wrapped(x, *args, **kwargs)  # 8-bit projections keep their own GEMMs between NCCL collectives
        a, b = gather_linear_multi(x, (ff.w1.weight, ff.w3.weight), group, "ffn-up")
        y = linear_reduce_scatter(swiglu(a, b), ff.w2.weight, group, "ffn-down")
        return y.view(x.shape)

    ff.forward = forward  # type: ignore[method-assign]


def shard_block_(block: nn.Module, tp_mesh) -> None:
    if getattr(block, "attention", None) is not None:
        block.attention.apply_tp(tp_mesh) if hasattr(block.attention, "apply_tp") else shard_attention_(block.attention, tp_mesh)
    ff = getattr(block, "feed_forward", None)
    if ff is not None:
        shard_feed_forward_(ff, tp_mesh)
    for name in ("attention_norm", "feed_forward_norm", "post_attention_norm", "post_feed_forward_norm"):
        _mark_partial(getattr(block, name, None), tp_mesh.get_group())
    moe = getattr(block, "feed_forward_moe", None)
    if moe is not None and hasattr(moe, "apply_tp"):
        moe.apply_tp(tp_mesh)


def shard_lm_head_(lm_head: nn.Module, tp_mesh) -> None:
    """
    Sequence-parallel head (the layout of src/olmo_core/nn/lm_head.py:366-417 with the fused loss): weights stay whole,
    every rank evaluates norm, projection and loss on its own ``T / tp`` tokens and the loss sums are added over the
    group. The parameters therefore see a sequence shard only: their gradients are partial sums.
    """
    group = tp_mesh.get_group()
    lm_head.tp_group = group
    _mark_partial(lm_head, group)


def shard_model_(model: nn.Module, tp_mesh) -> None:
    for block in model.blocks.values():
        block.apply_tp(tp_mesh)
    if getattr(model, "lm_head", None) is not None:
        model.lm_head.apply_tp(tp_mesh)
        head_weight = getattr(getattr(model.lm_head, "w_out", None), "weight", None)
        emb_weight = getattr(getattr(model, "embeddings", None), "weight", None)
        # A tied embedding shares the head's weight, whose gradient is a partial sum over the group: the embedding's
        # contribution has to be partial as well, or it would be counted once per rank.
        model._tp_embedding_partial = head_weight is not None and head_weight is emb_weight
        if model._tp_embedding_partial:
            _mark_partial(getattr(model, "embedding_norm", None), tp_mesh.get_group())
    # (an untied embedding and its norm are evaluated before the sequence is scattered: replicated, full gradients)
