"""CPU: partitioners and the vocabulary-sharded cross-entropy exchange, the latter with two gloo
ranks (world_size 2) where host implementations stand in for the CUDA kernels."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from oracle import ops as oracle


def test_shard_bounds_cover_and_balance():
    from arke_b200.sharding import shard_bounds
    for n in (0, 1, 7, 8, 8192, 128256):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)
    assert shard_bounds(128256, 8, 3) == (3 * 16032, 4 * 16032)


def test_attention_sharding_units_reassemble():
    from arke_b200.sharding import shard_attention
    q, k, v = oracle.make_attention_inputs(2, 8, 2, 32, 16, seed=1)
    outs = []
    for r in range(4):
        qf, kf, vf = shard_attention(q, k, v, 4, r)
        assert qf.shape == (1, 4, 32, 16) and kf.shape == (1, 1, 32, 16)
        outs.append(oracle.gqa_attention(qf, kf, vf, True))
    whole = oracle.gqa_attention(q, k, v, True)
    assert torch.equal(torch.cat(outs, dim=1).reshape(2, 8, 32, 16), whole)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arke_b200.sharding import combine_partials_reference, shard_bounds, vocab_sharded_ce
        x, w, labels = oracle.make_flce_inputs(96, 64, 1000, seed=7, ignore_frac=0.1)
        b, e = shard_bounds(w.shape[0], world, rank)
        tok, mean = vocab_sharded_ce(
            x, w[b:e], labels, b,
            partial_fn=lambda xx, ww, ll, off: oracle.ce_partials(xx, ww, ll, off),
            combine_fn=lambda pp, ll: combine_partials_reference(pp, ll))
        q.put((rank, tok.tolist(), float(mean)))  # plain lists: no shared-memory handles to outlive the child
    except Exception as exc:  # surface the failure instead of letting the parent time out
        q.put((rank, None, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_vocab_sharded_ce_two_gloo_ranks_match_unsharded():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, tok, mean in results:
        assert tok is not None, f"rank {rank} failed: {mean}"
    x, w, labels = oracle.make_flce_inputs(96, 64, 1000, seed=7, ignore_frac=0.1)
    tok_ref, mean_ref = oracle.fused_linear_ce(x, w, labels)
    for rank, tok, mean in results:
        assert torch.allclose(torch.tensor(tok), tok_ref, rtol=1e-5, atol=1e-5)
        assert abs(mean - mean_ref.item()) < 1e-5
    assert results[0][1] == results[1][1]      # identical on every rank


def _worker_bwd(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from arke_b200.sharding import lse_from_partials, shard_bounds, vocab_sharded_ce_backward
        x, w, labels = oracle.make_flce_inputs(64, 32, 500, seed=9, ignore_frac=0.1)
        b, e = shard_bounds(w.shape[0], world, rank)
        part = oracle.ce_partials(x, w[b:e], labels, b).contiguous()
        gathered = torch.empty((world * part.shape[0], 3), dtype=part.dtype)
        dist.all_gather_into_tensor(gathered, part)
        lse = lse_from_partials(gathered.view(world, -1, 3))
        dx, dw = vocab_sharded_ce_backward(
            x, w[b:e], labels, b, lse,
            backward_fn=lambda xx, ww, ll, ls, off: oracle.ce_backward_slice(xx, ww, ll, ls, off))
        q.put((rank, dx.tolist(), dw.tolist(), (b, e)))
    except Exception as exc:
        q.put((rank, None, repr(exc), None))
    finally:
        dist.destroy_process_group()


def test_vocab_sharded_backward_two_gloo_ranks_match_autograd():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_bwd, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    x, w, labels = oracle.make_flce_inputs(64, 32, 500, seed=9, ignore_frac=0.1)
    dx_ref, dw_ref = oracle.fused_linear_ce_backward(x, w, labels)
    for rank, dx, dw, be in results:
        assert dx is not None, f"rank {rank} failed: {dw}"
        assert torch.allclose(torch.tensor(dx), dx_ref, rtol=1e-4, atol=1e-7)          # summed over ranks
        assert torch.allclose(torch.tensor(dw), dw_ref[be[0]:be[1]], rtol=1e-4, atol=1e-7)   # own rows
    assert results[0][1] == results[1][1]


def test_ce_backward_slice_restatement_matches_autograd():
    x, w, labels = oracle.make_flce_inputs(48, 32, 300, seed=2, ignore_frac=0.2)
    from arke_b200.sharding import lse_from_partials
    lse = lse_from_partials(oracle.ce_partials(x, w, labels, 0))
    dx, dw = oracle.ce_backward_slice(x, w, labels, lse, 0, grad=0.5)
    dx_ref, dw_ref = oracle.fused_linear_ce_backward(x, w, labels)
    assert torch.allclose(dx, 0.5 * dx_ref, rtol=1e-4, atol=1e-7) and torch.allclose(dw, 0.5 * dw_ref, rtol=1e-4, atol=1e-7)


def _worker_leaves(rank, world, port, q):
    """Two steps of the vocabulary-sharded loss; rank 1 leaves between step 0 and step 1."""
    import datetime
    import time
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from arke_b200.sharding import (PeerLostError, StepLiveness, combine_partials_reference, shard_bounds,
                                    vocab_sharded_ce)
    live = StepLiveness.from_default_group(timeout_s=2.0)
    x, w, labels = oracle.make_flce_inputs(32, 16, 200, seed=3, ignore_frac=0.0)
    b, e = shard_bounds(w.shape[0], world, rank)
    step = lambda: vocab_sharded_ce(  # noqa: E731
        x, w[b:e], labels, b, partial_fn=lambda xx, ww, ll, off: oracle.ce_partials(xx, ww, ll, off),
        combine_fn=lambda pp, ll: combine_partials_reference(pp, ll))
    out = {"rank": rank}
    try:
        live.check_in(0)
        out["step0"] = float(step()[1])
        if rank == 1:
            q.put(out)                      # leaves between steps: nothing of its own in flight
            return                          # (no destroy_process_group: the process just ends)
        t0 = time.monotonic()
        try:
            live.check_in(1)
            out["step1"] = "check-in passed"
        except PeerLostError as exc:
            out["step1"] = ("peer_lost", exc.missing, round(time.monotonic() - t0, 2))
        # without the heartbeat the collective itself must end with an error, not hang
        t0 = time.monotonic()
        try:
            step()
            out["collective"] = "returned"
        except Exception as exc:            # gloo: RuntimeError (timeout / connection closed by peer)
            out["collective"] = ("error", type(exc).__name__, round(time.monotonic() - t0, 2))
        q.put(out)
    except Exception as exc:
        out["fatal"] = repr(exc)
        q.put(out)


def test_rank_leaving_between_steps_is_an_error_in_bounded_time_not_a_hang():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker_leaves, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        r = q.get(timeout=90)
        results[r["rank"]] = r
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode is not None          # nobody hangs
    assert "fatal" not in results[0] and "fatal" not in results[1], results
    assert abs(results[0]["step0"] - results[1]["step0"]) < 1e-6          # the step before the loss worked
    kind, missing, secs = results[0]["step1"]
    assert kind == "peer_lost" and missing == [1] and secs < 10
    assert results[0]["collective"][0] == "error" and results[0]["collective"][2] < 30, results[0]
