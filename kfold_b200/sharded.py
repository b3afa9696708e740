"""Row-sharded pair track across the GPUs of one node (one process per GPU, torch.distributed / NCCL).

The reference never splits a pair tensor: its multi-GPU mode hands whole complexes to different GPUs
(src/kfold/cli/multigpu.py:22-77).  For complexes too large or too slow for one GPU this module shards the
pair representation z (N, N, C) by rows: rank r owns rows [r*N/P, (r+1)*N/P).  Per operator:

  pointwise (LayerNorm, projections, gates, transition, residual)   local
  triangle multiplication, outgoing   t[i,j] = sum_k a[i,k] b[j,k]    the contraction is independent per channel:
                                      ALL-TO-ALL of a and b to a channel-sharded layout (every rank gets all rows of
                                      C/P channels), local contraction, ALL-TO-ALL of t back to row shards.  That moves
                                      3 N^2 C / P values per rank instead of the (P-1) N^2 C / P of an all-gather of b
                                      (the all-gather form is kept below four ranks and for C not divisible by P)
  triangle multiplication, incoming   t[i,j] = sum_k a[k,i] b[k,j]    channel-sharded form: the projection writes a, b
                                      transposed ([i][k], k = the rank's own rows), the all-to-all leaves K in one piece
                                      per source rank and the contraction walks the pieces: z itself is never transposed.
                                      All-gather form: a, b are taken from the TRANSPOSED shard (all-to-all transpose of
                                      z), where it is the outgoing form; the output gate and the residual use the row shard
  triangle attention, starting node   rows local; ALL-GATHER of the projected triangle bias only (N*N*H)
  triangle attention, ending node     starting node on the transposed shard, result transposed back; the three reorders
                                      around the two all-to-alls ride in the LayerNorm, the projection's operand strides and
                                      the output projection's store strides
  single track / pair bias            bias rows stay local: every rank attends with its own rows as queries (cross form) and the
                                      updated rows of the replicated single track are all-gathered

Everything here is host-side orchestration: the kernels are the same ones the single-GPU path uses, called
through the two-phase C entry points (kfb_trimul_project / _finish, kfb_triatt_project / _finish).
The data movement helpers (`transpose_shard`, `gather_rows`) work on CPU tensors with the gloo backend too,
which is how they are unit-tested.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _lib as L
from . import functional as F
from . import packing


# NCCL's point-to-point transport (what an all-to-all is made of) uses few channels by default: on two B200s a 268 MB
# all-to-all ran at 323 GB/s per rank with the defaults and at 550 GB/s with these (the all-gather is unaffected).
NCCL_ENV_DEFAULTS = {"NCCL_MIN_P2P_NCHANNELS": "64", "NCCL_MAX_P2P_NCHANNELS": "64", "NCCL_MIN_NCHANNELS": "32"}


def apply_nccl_env_defaults() -> None:
    """Set the NCCL variables above unless the user already chose values.  Call before the process group is created."""
    import os
    for k, v in NCCL_ENV_DEFAULTS.items():
        os.environ.setdefault(k, v)


def shard_rows(n: int, world: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the rows rank `rank` owns; n must divide evenly (pad the complex otherwise)."""
    if n % world != 0:
        raise ValueError(f"N={n} is not divisible by the number of ranks {world}")
    rows = n // world
    return rank * rows, (rank + 1) * rows


def transpose_shard(x_loc: torch.Tensor, group=None, add_to: torch.Tensor | None = None) -> torch.Tensor:
    """Row shard of z -> row shard of z^T with one all-to-all.

    x_loc (rows, N, *tail) holds z[r*rows : (r+1)*rows, :]; the result holds z^T[r*rows : (r+1)*rows, :],
    i.e. out[i, k] = z[k, r*rows + i].  With `add_to` (same shape as the result) the sum add_to + z^T shard is
    returned, formed in the pass that reorders the received blocks.
    """
    world = dist.get_world_size(group)
    rows, n = x_loc.shape[0], x_loc.shape[1]
    tail = x_loc.shape[2:]
    if rows * world != n:
        raise ValueError(f"shard of {rows} rows x {n} columns does not match {world} ranks")
    # send[q] = the block of my rows that lies in rank q's columns
    send = x_loc.reshape(rows, world, rows, *tail).transpose(0, 1).contiguous()      # [q][i_loc][j_q]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[q][i_q][j_loc] = z[q*rows + i_q, r*rows + j_loc]  ->  out[j_loc][q*rows + i_q]
    if add_to is not None:
        return add_to + recv.permute(2, 0, 1, *range(3, recv.dim())).reshape(rows, n, *tail)
    return recv.permute(2, 0, 1, *range(3, recv.dim())).reshape(rows, n, *tail).contiguous()


def gather_rows(x_loc: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather along the first dimension: (rows, ...) on every rank -> (world*rows, ...)."""
    world = dist.get_world_size(group)
    out = torch.empty((world * x_loc.shape[0],) + tuple(x_loc.shape[1:]), dtype=x_loc.dtype, device=x_loc.device)
    dist.all_gather_into_tensor(out, x_loc.contiguous(), group=group)
    return out


def gather_head_rows(x_loc: torch.Tensor, group=None) -> torch.Tensor:
    """(H, rows, n) on every rank -> (H, world*rows, n) with ONE all-gather and one local permute.

    The gathered buffer arrives rank after rank, [world][H][rows][n]; the attention kernels want each head's rows in
    their natural order, so the heads are moved to the front afterwards (a copy of N*N*H values, far cheaper than one
    collective per head)."""
    world = dist.get_world_size(group)
    h, rows, n = x_loc.shape
    buf = torch.empty((world * h, rows, n), dtype=x_loc.dtype, device=x_loc.device)
    dist.all_gather_into_tensor(buf, x_loc.contiguous(), group=group)
    return buf.view(world, h, rows, n).permute(1, 0, 2, 3).reshape(h, world * rows, n).contiguous()


def _bf16(shape, device):
    return torch.empty(shape, dtype=torch.bfloat16, device=device)


class ShardedPairOps:
    """The pair-track operators on a row shard.  `group` is the process group whose ranks share one complex."""

    def __init__(self, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._mask_t = None   # (key, transposed mask shard): the pair mask of a complex is the same for every block

    def _transposed_mask(self, mask_loc: torch.Tensor) -> torch.Tensor:
        """Row shard of the transposed pair mask, exchanged once per mask tensor and reused by every later call."""
        key = (mask_loc.data_ptr(), None if torch.is_inference(mask_loc) else mask_loc._version, tuple(mask_loc.shape),
               mask_loc.dtype)
        if self._mask_t is None or self._mask_t[0] != key:
            # the cache keeps `mask_loc` alive so that its address cannot be reused by another tensor
            self._mask_t = (key, transpose_shard(mask_loc.to(torch.uint8), self.group), mask_loc)
        return self._mask_t[1]

    # ------------------------------------------------------------------ triangle multiplication
    def _trimul_cs(self, x_loc: torch.Tensor, mask_loc: torch.Tensor, pk: dict, eps: float, incoming: bool):
        """Channel-sharded exchange, either direction, from the row shard alone.  `pk` must come from
        pack_trimul(..., shard_world=world, shard_parts=parts): the projection then writes the operand channels group by
        group and rank by rank, [h][q][a, b][C/(parts P)], each group the send buffer of an all-to-all as it lies.  The
        incoming direction projects with the transposed walk (a[k][i] stored at [i][k]) and contracts over a K that lies
        in one piece per source rank: no transpose of z.  With two groups the exchanges of one run under the projection
        and the contraction of the other."""
        rows, n, c = x_loc.shape
        world, parts = self.world, pk.get("shard_parts", 1)
        cl = c // (world * parts)
        dev = x_loc.device
        lib = L.lib()
        dt = L.dtype_code(x_loc.dtype)
        xn = _bf16((rows * n, c), dev)
        gl = _bf16((rows * n, c), dev)
        m8 = mask_loc.to(torch.bool).contiguous().view(torch.uint8)
        x_loc = x_loc.contiguous()
        tr = 1 if incoming else 0
        shape = (world, 2, cl, n, rows) if incoming else (world, 2, cl, rows, n)
        t = _bf16((parts, world, cl, rows, n), dev)          # = t [c][rows][n] in the original channel order
        with L.on_device(dev):
            st = L.stream_ptr()
            sends, recvs, works = [], [], []
            for h in range(parts):
                ab = _bf16(shape, dev)
                L.check(lib.kfb_trimul_project(L.ptr(x_loc) if h == 0 else None, L.ptr(m8), L.ptr(pk["ln_in_w"]), L.ptr(pk["ln_in_b"]),
                                               L.ptr(pk["w_in"]), None, L.ptr(xn), L.ptr(ab), None, 1, rows, n, c, tr, h, parts, eps,
                                               dt, st))
                ab_recv = torch.empty_like(ab)
                works.append(dist.all_to_all_single(ab_recv, ab, group=self.group, async_op=True))   # [source rank][a, b][cl]..
                sends.append(ab)
                recvs.append(ab_recv)
            # the output-gate logits, from the rows normalised above, while the exchanges are in flight
            L.check(lib.kfb_trimul_project(None, None, None, None, None, L.ptr(pk["w_gout"]), L.ptr(xn), None, L.ptr(gl), 1, rows,
                                           n, c, 0, 0, 1, eps, dt, st))
            back = []
            for h in range(parts):
                works[h].wait()
                t_send = _bf16((world, cl, rows, n), dev)
                L.check(lib.kfb_trimul_contract_cs(L.ptr(recvs[h]), L.ptr(t_send), world, rows, n, cl, tr, st))
                back.append((dist.all_to_all_single(t[h], t_send, group=self.group, async_op=True), t_send))
            for work, _ in back:
                work.wait()
            out = torch.empty_like(x_loc)
            L.check(lib.kfb_trimul_finish(None, None, rows, 0, L.ptr(gl), L.ptr(pk["ln_out_w"]), L.ptr(pk["ln_out_b"]),
                                          L.ptr(pk["w_pout"]), L.ptr(t), L.ptr(xn), L.ptr(out), L.ptr(x_loc), rows, n, c, eps,
                                          dt, st))
        return out

    def _trimul(self, x_ab: torch.Tensor, mask_ab: torch.Tensor, x_row: torch.Tensor, pk: dict, eps: float):
        """All-gather form: a, b from (x_ab, mask_ab); gate logits and residual from x_row.  All (rows, N, ...) shards.
        Operand b is projected first and gathered in two channel halves; a and the gate logits are projected, and the
        first half contracted, while the gathers are in flight."""
        rows, n, c = x_row.shape
        dev = x_row.device
        lib = L.lib()
        dt = L.dtype_code(x_row.dtype)
        xn = _bf16((rows * n, c), dev)
        ab = _bf16((2 * c, rows, n), dev)
        gl = _bf16((rows * n, c), dev)
        m8 = mask_ab.to(torch.bool).contiguous().view(torch.uint8)
        x_ab = x_ab.contiguous()
        x_row = x_row.contiguous()
        split = c % 128 == 0              # the projection then divides into whole tiles per operand, the channels into halves
        rn = rows * n
        with L.on_device(dev):
            st = L.stream_ptr()
            same = x_ab.data_ptr() == x_row.data_ptr()
            if not split:
                L.check(lib.kfb_trimul_project(L.ptr(x_ab), L.ptr(m8), L.ptr(pk["ln_in_w"]), L.ptr(pk["ln_in_b"]), L.ptr(pk["w_in"]),
                                               None, L.ptr(xn), L.ptr(ab), None, 1, rows, n, c, 0, 0, 1, eps, dt, st))
                halves = [(0, c)]
            else:
                L.check(lib.kfb_trimul_project(L.ptr(x_ab), L.ptr(m8), L.ptr(pk["ln_in_w"]), L.ptr(pk["ln_in_b"]), L.ptr(pk["w_in"]),
                                               None, L.ptr(xn), L.ptr(ab[c:]), None, 1, rows, n, c, 0, 1, 2, eps, dt, st))
                halves = [(0, c // 2), (c // 2, c)]
            gathers = []
            for lo, hi in halves:      # [world][channels of the half][rows][n], rank after rank
                b_full = torch.empty((self.world * (hi - lo), rows, n), dtype=torch.bfloat16, device=dev)
                gathers.append((dist.all_gather_into_tensor(b_full, ab[c + lo:c + hi], group=self.group, async_op=True), b_full))
            if split:
                L.check(lib.kfb_trimul_project(None, L.ptr(m8), None, None, L.ptr(pk["w_in"]), None, L.ptr(xn), L.ptr(ab), None, 1,
                                               rows, n, c, 0, 0, 2, eps, dt, st))
            L.check(lib.kfb_trimul_project(None if same else L.ptr(x_row), None, L.ptr(pk["ln_in_w"]), L.ptr(pk["ln_in_b"]), None,
                                           L.ptr(pk["w_gout"]), L.ptr(xn), None, L.ptr(gl), 1, rows, n, c, 0, 0, 1, eps, dt, st))
            t = _bf16((c, rows, n), dev)
            for (lo, hi), (work, b_full) in zip(halves, gathers):
                work.wait()
                L.check(lib.kfb_trimul_contract(L.ptr(ab[lo:hi]), L.ptr(b_full), rows, (hi - lo) * rn, L.ptr(t[lo:hi]), rows, n,
                                                hi - lo, st))
            out = torch.empty_like(x_row)
            L.check(lib.kfb_trimul_finish(None, None, rows, 0, L.ptr(gl), L.ptr(pk["ln_out_w"]), L.ptr(pk["ln_out_b"]),
                                          L.ptr(pk["w_pout"]), L.ptr(t), L.ptr(xn), L.ptr(out), L.ptr(x_row), rows, n, c, eps, dt,
                                          st))
        return out

    def _channel_form(self, pk: dict, rows: int) -> bool:
        return pk.get("shard_world", 0) == self.world and self.world > 1 and rows % 64 == 0

    def trimul_outgoing(self, x_loc, mask_loc, pk, eps: float = 1e-5):
        """x + TriangleMultiplicationOutgoing(x) on the row shard (rows, N, C); mask_loc (rows, N)."""
        if self._channel_form(pk, x_loc.shape[0]):
            return self._trimul_cs(x_loc, mask_loc, pk, eps, incoming=False)
        return self._trimul(x_loc, mask_loc, x_loc, pk, eps)

    def trimul_incoming(self, x_loc, mask_loc, pk, eps: float = 1e-5):
        """x + TriangleMultiplicationIncoming(x): with the channel-sharded exchange straight from the row shard, otherwise
        with the operands taken from the transposed shard."""
        if self._channel_form(pk, x_loc.shape[0]):
            return self._trimul_cs(x_loc, mask_loc, pk, eps, incoming=True)
        if pk.get("shard_world", 0):
            raise ValueError("trimul_incoming: weights packed for the channel exchange need shards of a multiple of 64 rows")
        xt = transpose_shard(x_loc, self.group)
        return self._trimul(xt, self._transposed_mask(mask_loc), x_loc, pk, eps)

    # ------------------------------------------------------------------ triangle attention
    def _triatt_start(self, x_loc, mask_loc, pk, eps: float, resid: bool):
        rows, n, c = x_loc.shape
        heads = pk["heads"]
        dp = packing.head_dim_pad(c // heads)
        hdp = heads * dp
        dev = x_loc.device
        lib = L.lib()
        dt = L.dtype_code(x_loc.dtype)
        x_loc = x_loc.contiguous()
        xn = _bf16((rows * n, c), dev)
        qkg = _bf16((rows * n, 3 * hdp), dev)
        vt = _bf16((rows, hdp, n), dev)
        bias_loc = _bf16((heads, rows, n), dev)
        m8 = mask_loc.to(torch.bool).contiguous().view(torch.uint8)
        with L.on_device(dev):
            L.check(lib.kfb_triatt_project(L.ptr(x_loc), L.ptr(pk["ln_w"]), L.ptr(pk["ln_b"]), L.ptr(pk["w_proj"]), L.ptr(xn),
                                           L.ptr(qkg), L.ptr(vt), L.ptr(bias_loc), rows, n, c, heads, 0, eps, dt, L.stream_ptr()))
            bias_full = gather_head_rows(bias_loc, self.group)
            out = torch.empty_like(x_loc)
            L.check(lib.kfb_triatt_finish(L.ptr(qkg), L.ptr(vt), L.ptr(bias_full), L.ptr(m8), L.ptr(pk["w_out"]), L.ptr(xn),
                                          L.ptr(out), L.ptr(x_loc) if resid else None, rows, n, c, heads, 0, dt, L.stream_ptr()))
        return out

    def triatt_starting(self, x_loc, mask_loc, pk, eps: float = 1e-5):
        return self._triatt_start(x_loc, mask_loc, pk, eps, resid=True)

    def triatt_ending(self, x_loc, mask_loc, pk, eps: float = 1e-5):
        """x + TriangleAttentionEndingNode(x): the starting-node operator on the transposed shard.  LayerNorm runs before
        the transpose and writes the all-to-all's send buffer; the projection reads the received buffer as it lies, the
        output projection writes the update as the send buffer of the transpose back: three kernels carry the reorders
        that would otherwise be three copies of the shard."""
        rows, n, c = x_loc.shape
        world = self.world
        heads = pk["heads"]
        hdp = heads * packing.head_dim_pad(c // heads)
        dev = x_loc.device
        lib = L.lib()
        bf = L.dtype_code(torch.bfloat16)
        x_loc = x_loc.contiguous()
        m8 = self._transposed_mask(mask_loc).to(torch.bool).contiguous().view(torch.uint8)
        send = _bf16((world, rows, rows, c), dev)
        recv = torch.empty_like(send)
        qkg = _bf16((rows * n, 3 * hdp), dev)
        vt = _bf16((rows, hdp, n), dev)
        bias_loc = _bf16((heads, rows, n), dev)
        with L.on_device(dev):
            L.check(lib.kfb_layernorm_exchange(L.ptr(x_loc), L.ptr(send), L.ptr(pk["ln_w"]), L.ptr(pk["ln_b"]), rows, n, c, eps,
                                               L.dtype_code(x_loc.dtype), L.stream_ptr()))
            dist.all_to_all_single(recv, send, group=self.group)      # recv[q][i_q][j] = LN(z)[q*rows + i_q][r*rows + j]
            L.check(lib.kfb_triatt_project(L.ptr(recv), None, None, L.ptr(pk["w_proj"]), None, L.ptr(qkg), L.ptr(vt),
                                           L.ptr(bias_loc), rows, n, c, heads, 1, eps, bf, L.stream_ptr()))
            bias_full = gather_head_rows(bias_loc, self.group)
            # `send` is free again (the exchange has read it): attention output; `recv` (read by the projection): the update
            L.check(lib.kfb_triatt_finish(L.ptr(qkg), L.ptr(vt), L.ptr(bias_full), L.ptr(m8), L.ptr(pk["w_out"]), L.ptr(send),
                                          L.ptr(recv), None, rows, n, c, heads, 1, bf, L.stream_ptr()))
            upd = torch.empty_like(recv)
            dist.all_to_all_single(upd, recv, group=self.group)       # upd[q][j][i] = update of z[r*rows + i][q*rows + j]
        return x_loc + upd.permute(2, 0, 1, 3).reshape(rows, n, c)

    # ------------------------------------------------------------------ pair bias for the single track
    def pair_bias(self, x_loc, ln_w, ln_b, w, eps: float = 1e-5):
        """(H, N, N) bias from the row shard: local projection, then all-gather per head."""
        rows, n, c = x_loc.shape
        heads = w.shape[0]
        # the 1-GPU op expects square tensors; project the shard as `rows` independent 1 x n rows
        loc = F.pair_bias_rows(x_loc, ln_w, ln_b, w, eps)                     # (heads, rows, n)
        return gather_head_rows(loc, self.group)


class ShardedPairformerBlock:
    """The composite Pairformer block on a row shard.  Wraps the weights of a `modules.PairformerBlock`."""

    def __init__(self, block, group=None, exchange: str = "auto"):
        """``exchange``: how the triangle multiplication moves its operands: "channel" (all-to-all to a channel-sharded
        layout), "gather" (all-gather of b) or "auto" (channel from four ranks on)."""
        if exchange not in ("auto", "channel", "gather"):
            raise ValueError(f"unknown exchange {exchange!r}")
        self.block = block
        self.ops = ShardedPairOps(group)
        self.exchange = exchange
        self._trimul_packs = {}
        self._apb_cross_pack = None

    def _pack_trimul(self, mod, dev, rows: int, incoming: bool):
        """Weights for the channel-sharded exchange when C divides by the number of ranks (packed once per module)."""
        world = self.ops.world
        c = mod.layernorm_in.normalized_shape
        # outgoing: the channel-sharded exchange moves 3 N^2 C / P values per rank, the all-gather of b (P - 1) N^2 C / P: it
        # pays from four ranks on.  Incoming: the all-gather form also transposes z, the channel form does not: it pays always.
        channel = self.exchange == "channel" or (self.exchange == "auto" and (world >= 4 or incoming))
        if world == 1 or not channel or c % world != 0 or rows % 64 != 0:
            return mod._packed(dev, torch.bfloat16, packing.pack_trimul)
        key = (id(mod), dev)
        if key not in self._trimul_packs:
            parts = 2 if (c % 128 == 0 and (c // world) % 2 == 0) else 1     # two exchange groups when the tiles divide
            pk = packing.pack_trimul(mod.state_dict(), dev, shard_world=world, shard_parts=parts)
            pk["shard_world"], pk["shard_parts"] = world, parts
            self._trimul_packs[key] = pk
        return self._trimul_packs[key]

    @torch.no_grad()
    def __call__(self, z_loc: torch.Tensor, s: torch.Tensor, pair_mask_loc: torch.Tensor, mask: torch.Tensor):
        """z_loc (rows, N, c_z) row shard; s (1, N, c_s) replicated; pair_mask_loc (rows, N); mask (1, N)."""
        b, ops = self.block, self.ops
        dev = z_loc.device
        bf = torch.bfloat16
        rows = z_loc.shape[0]
        z = ops.trimul_outgoing(z_loc, pair_mask_loc, self._pack_trimul(b.tri_mul_out, dev, rows, False))
        z = ops.trimul_incoming(z, pair_mask_loc, self._pack_trimul(b.tri_mul_in, dev, rows, True))
        pk_s = b.tri_att_start._packed(dev, bf, lambda sd, d: packing.pack_triatt(sd, b.tri_att_start.no_heads, d))
        pk_e = b.tri_att_end._packed(dev, bf, lambda sd, d: packing.pack_triatt(sd, b.tri_att_end.no_heads, d))
        z = ops.triatt_starting(z, pair_mask_loc, pk_s)
        z = ops.triatt_ending(z, pair_mask_loc, pk_e)
        z = b.transition_z(z, residual=True)
        s = self._single_track(z, s, mask)
        s = b.transition(s, residual=True)
        return z, s

    def _single_track(self, z_loc: torch.Tensor, s: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """s + SelfAttentionPairBias(s, bias from z): the single track is replicated, but its pair bias is not: every rank
        projects the bias of its own rows, attends with its own rows as queries against all tokens as keys (the cross
        form of the kernel) and the updated rows are all-gathered -- N x c_s values instead of the H x N x N bias."""
        b, ops = self.block, self.ops
        att = b.attention
        dev = z_loc.device
        bf = torch.bfloat16
        rows, n, _ = z_loc.shape
        if ops.world == 1 or rows % 8 != 0 or s.shape[0] != 1:
            bias = ops.pair_bias(z_loc, b.layernorm_z.weight.detach().float(), b.layernorm_z.bias.detach().float(),
                                 b.linear_pair_bias.weight.detach().to(dev, bf).contiguous(), b.layernorm_z.eps)
            return att(s, None, bias.unsqueeze(0), mask, residual=True)
        key = (id(att), dev)
        if self._apb_cross_pack is None or self._apb_cross_pack[0] != key:
            self._apb_cross_pack = (key, packing.pack_apb_cross(att.state_dict(), att.num_heads, dev))
        pk = self._apb_cross_pack[1]
        r0 = ops.rank * rows
        bias_loc = F.pair_bias_rows(z_loc, b.layernorm_z.weight.detach().float(), b.layernorm_z.bias.detach().float(),
                                    b.linear_pair_bias.weight.detach().to(dev, bf).contiguous(), b.layernorm_z.eps)   # (H, rows, N)
        ln = att.layernorm_a
        an = F.layer_norm(s, ln.weight, ln.bias, ln.eps, out_dtype=bf)                                              # (1, N, c_s)
        upd = F.attention_pair_bias_cross(an[:, r0:r0 + rows].contiguous(), an, bias_loc.unsqueeze(0), mask.reshape(1, n), pk,
                                          out_dtype=s.dtype, resid=s[:, r0:r0 + rows].contiguous())                # (1, rows, c_s)
        return gather_rows(upd[0], ops.group).unsqueeze(0)
