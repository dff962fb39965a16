"""Expert-parallel layer over 1/2/4/8 GPUs of one node (one process per GPU, torch.distributed for the plumbing).

The reference shards every expert four ways by tensor parallelism and, after each MoE layer, all-gathers the
ranks' fp32 partial outputs and adds them in fixed rank order (src/model.rs:485-496, src/comm.rs:1-2: "never sum
in NCCL").  Here the shards are whole experts:
  * routed expert e lives on rank e // (experts / world)              (contiguous windows)
  * the shared expert (every row uses it): windows of <= 16 rows -- owned by rank  layer % world  (round robin over
    the layers; the rule the planning functions below model), or, with dynamic_shared=True, decided window by window on
    the device: the rank whose experts the window's routing table uses least (fewest distinct, ties to the lowest rank)
    takes it; larger windows (prefill) -- split by ROWS, rank k computes it for rows [k, k+1) * ceil(max_rows / world)
  * grouping runs on every rank from the replicated picks (deterministic, so the ranks agree without talking)
  * each rank computes the pairs of its window and combines them into a partial out_g[rows][hidden] fp32
  * exchange = all-gather of the partials over NVLink (NCCL) + the same fixed rank-order sum as the reference
The planning functions are pure python so that they are tested on CPU ranks (gloo) with the oracle as compute.
"""


def expert_window(rank, world, experts):
    """[lo, hi) of routed expert ids computed on `rank`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank outside the world")
    if experts % world:
        raise ValueError("the number of routed experts must be divisible by the world size")
    per = experts // world
    return rank * per, (rank + 1) * per


def shared_owner(layer, world):
    """Rank that computes the shared expert of `layer`."""
    return layer % world


def shared_rows(rank, world, max_rows):
    """[lo, hi) of window rows whose shared-expert pair `rank` computes in a handle for more than 16 rows."""
    per = -(-max_rows // world)
    return rank * per, (rank + 1) * per


def computed_here(picks, rank, world, experts, layer, max_rows=None):
    """Boolean mask [rows][slots]: which pairs this rank computes (the library's window rule).  max_rows: the handle's
    row capacity; above 16 the shared expert is split by rows instead of going to one rank per layer."""
    import numpy as np
    lo, hi = expert_window(rank, world, experts)
    picks = np.asarray(picks)
    routed = (picks >= lo) & (picks < hi) & (picks < experts)
    if max_rows is not None and max_rows > 16 and world > 1:
        rlo, rhi = shared_rows(rank, world, max_rows)
        rows = np.arange(picks.shape[0])[:, None]
        shared = (picks == experts) & (rows >= rlo) & (rows < rhi)
    else:
        shared = (picks == experts) & (shared_owner(layer, world) == rank)
    return routed | shared


class ExchangeError(RuntimeError):
    """A rank did not take part in an exchange (it failed, or never arrived), or the collective itself failed."""


def arrive(store, step, rank, world, timeout_s=5.0):
    """Host-side agreement before exchange `step`: no rank enters the collective unless every rank has arrived (the
    reference agrees across ranks before its first exchange, src/roce.rs:235-273, and closes a failed transfer group
    instead of leaving peers inside it, src/nccl_exchange_plan.rs:163-197).  `store`: a torch.distributed store.  A rank
    that cannot take part calls withdraw(); its peers then raise ExchangeError at once, and after `timeout_s` when a
    rank simply never arrives -- nobody is left hanging inside a collective."""
    import datetime
    import time
    store.set(f"ep/{step}/{rank}", b"ok")
    deadline = time.monotonic() + timeout_s
    for k in range(world):
        left = max(0.05, deadline - time.monotonic())
        try:
            store.wait([f"ep/{step}/{k}"], datetime.timedelta(seconds=left))
        except Exception as ex:                                # the store's time-out
            raise ExchangeError(f"rank {k} did not reach exchange {step} within {timeout_s} s") from ex
        word = bytes(store.get(f"ep/{step}/{k}"))
        if word != b"ok":
            raise ExchangeError(f"rank {k} withdrew from exchange {step}: {word.decode(errors='replace')}")


def withdraw(store, step, rank, why):
    """Tell the peers that this rank will not take part in exchange `step` (see arrive)."""
    store.set(f"ep/{step}/{rank}", ("failed: " + str(why)).encode())


def exchange(partial, gathered, out, group=None, rank_sum=None, all_gather=None):
    """All-gather `partial` [rows][H] fp32 into `gathered` [world][rows][H] and add the ranks' rows in ascending
    rank order into `out`.  A failing collective surfaces as ExchangeError.  `rank_sum(gathered, out)` is the device kernel (glmflash_rank_sum) on GPUs; on CPU
    ranks the same ordered sum is done with torch."""
    import torch.distributed as dist
    try:
        if all_gather is not None:                             # injectable, as the reference's plan takes its NCCL calls as closures
            all_gather(gathered.view(-1), partial.reshape(-1))
        else:
            dist.all_gather_into_tensor(gathered.view(-1), partial.reshape(-1), group=group)
    except ExchangeError:
        raise
    except Exception as ex:
        raise ExchangeError(f"all-gather of the partial layer outputs failed: {ex}") from ex
    if rank_sum is not None:
        rank_sum(gathered, out)
    else:
        acc = gathered[0].clone()
        for k in range(1, gathered.shape[0]):
            acc += gathered[k]
        out.copy_(acc)
    return out


class EpMoe:
    """One MoE layer call, expert parallel: Moe handles with this rank's window (with and without the shared
    expert) and run(layer, ...) -> final [rows][H] on every rank.
    exchange = "nvlink": the library's fused combine + NVLink push + ordered sum kernel (glmflash_ep_combine);
    exchange = "nccl":   local combine, NCCL all-gather of the partials, rank-ordered sum kernel (the baseline)."""

    def __init__(self, pkg, rank, world, max_rows, hidden=2048, inter=1536, experts=64, slots=5, group=None, device=None,
                 exchange="nvlink", dynamic_shared=None):
        import torch
        import torch.distributed as dist
        self.pkg, self.rank, self.world, self.group = pkg, rank, world, group
        self.experts, self.hidden, self.exchange = experts, hidden, exchange if world > 1 else "none"
        lo, hi = expert_window(rank, world, experts)
        self.window = (lo, hi)
        self.row_split = world > 1 and max_rows > 16           # prefill: the shared expert is split by rows
        srows = shared_rows(rank, world, max_rows) if self.row_split else (0, 0)
        # windows of <= 16 rows: the shared expert goes round robin over the layers; dynamic_shared=True: window by window to
        # the rank with the fewest routed experts of that window (decided on the device, config shared_exl3 = 2) -- measured
        # on 2 GPUs the decision costs about as much as the better balance gains (28.3 vs 27.2 us per one-token layer)
        self.dynamic = bool(dynamic_shared) and world > 1 and not self.row_split
        kinds = (1,) if world == 1 or self.row_split else ((2,) if self.dynamic else (0, 1))
        self.moes = {sh: pkg.Moe(pkg.make_config(hidden, inter, experts, slots, max_rows=max_rows, shared_exl3=sh,
                                                 expert_lo=lo, expert_hi=hi, shared_rows=srows)) for sh in kinds}
        if self.exchange == "nccl":
            self.gathered = torch.empty((world, max_rows, hidden), dtype=torch.float32, device=device)
            self.final = torch.empty((max_rows, hidden), dtype=torch.float32, device=device)
        elif self.exchange == "nvlink":
            def gather(local):
                out = [None] * world
                dist.all_gather_object(out, local, group=group)
                return out
            cfg = pkg.make_config(hidden, inter, experts, slots, max_rows=max_rows, shared_exl3=0, expert_lo=lo, expert_hi=hi,
                                  shared_rows=srows)
            self.ep = pkg.EpCombine(cfg, rank, world, gather)

    def owns_shared(self, layer):
        """1 / 0: this rank computes / skips the shared expert of this layer; 2: decided per window on the device."""
        if self.dynamic:
            return 2
        return int(self.world == 1 or self.row_split or shared_owner(layer, self.world) == self.rank)

    def owner(self, layer):
        return self.moes[self.owns_shared(layer)]

    def run(self, layer, w, x, picks, route_w, rows, out=None, stream=None):
        m = self.owner(layer)
        if self.exchange == "nvlink":
            # one call: the layer and its exchange (windows of <= 16 rows: one launch per rank)
            res = m.run_ep(self.ep, w, x, picks, route_w, rows, shared_here=self.owns_shared(layer), stream=stream)
            if out is not None:
                out.copy_(res)
                return out
            return res
        m.run(w, x, picks, route_w, rows, stream=stream)
        if self.exchange == "none":
            return m.output[:rows]
        out = self.final[:rows] if out is None else out
        g = self.gathered if rows == self.gathered.shape[1] else \
            self.gathered.view(-1)[: self.world * rows * self.hidden].view(self.world, rows, self.hidden)
        return exchange(m.output[:rows], g, out, self.group, lambda a, b: self.pkg.rank_sum(a, b, stream=stream))

    def check(self):
        """Raises when a bounded wait inside a kernel gave up since the last check (call after synchronising)."""
        import torch
        torch.cuda.synchronize()
        bad = {k: int(m.status.cpu()[0]) for k, m in self.moes.items() if int(m.status.cpu()[0])}
        if self.exchange == "nvlink" and int(self.ep.status.cpu()[0]):
            bad["exchange"] = int(self.ep.status.cpu()[0])
        if bad:
            raise self.pkg.GlmFlashError(f"device status words are set: {bad}")
