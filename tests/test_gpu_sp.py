"""Sequence-parallel path on the CUDA kernels: the shards of one packed sequence are run as host
threads of one process on one GPU (only host threads wait for each other; no kernel waits on
another), and the result is compared with the unsharded operator and with the CPU oracle."""
import threading

import pytest
import torch

from oracle import delta_oracle as O

pytestmark = pytest.mark.gpu


def _run_sharded(n, ins, seg, init, do, dfs, exchange="gather", **opts):
    from deltanet_b200 import sp
    chains = sp.LocalChain.make(n)
    L = ins[0].shape[1]
    results, errors = [None] * n, []

    def work(r):
        try:
            lo, hi = r * L // n, (r + 1) * L // n
            # sp_forward / sp_backward are what chunk_gdn2_sp's autograd node calls.  They are called
            # directly here because torch runs all CUDA backward nodes of a process on ONE engine
            # thread, where two emulated ranks would wait for each other forever.
            shard = [t[:, lo:hi].contiguous() for t in ins]
            ops = sp.CudaOps(**opts)
            out, final, c = sp.sp_forward(ops, chains[r], shard, seg[:, lo:hi].contiguous(), init if r == 0 else None, exchange)
            grads, d_in = sp.sp_backward(ops, chains[r], c, do[:, lo:hi].contiguous(), dfs if r == n - 1 else None)
            results[r] = dict(out=out, final=final, grads=list(grads) + [d_in])
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=work, args=(r,)) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not errors, errors
    return results


@pytest.mark.parametrize("n,prec,C,K,V,tol,recompute", [
    (2, "fp32", 64, 64, 64, 2e-4, False), (4, "fp32", 64, 64, 64, 2e-4, True),
    (2, "bf16", 128, 128, 128, 2e-2, False), (4, "bf16", 128, 128, 128, 2e-2, False),
    (4, "bf16", 64, 128, 128, 2e-2, True)])                 # chunk 64 + recompute_states: the long-sequence configuration's settings
def test_sharded_equals_unsharded(n, prec, C, K, V, tol, recompute):
    """Shards with no boundary, with one, and with several, so that the correction passes stop at the
    first / last boundary of a shard, run through a whole shard, and are skipped where a shard starts a
    document."""
    import deltanet_b200 as dn
    B, L, Hk, Hv = 2, 1024, 2, 4
    q, k, v, g, b, w = O.make_inputs(91, B, L, Hk, Hv, K, V, qkv_scale=0.5)
    seg = torch.stack([torch.repeat_interleave(torch.tensor([0, 1, 2], dtype=torch.int32), torch.tensor([300, 212, 512])),
                       torch.repeat_interleave(torch.tensor([7, 8, 9, 10], dtype=torch.int32), torch.tensor([256, 256, 100, 412]))])
    gen = torch.Generator().manual_seed(5)
    init = torch.randn(B, Hv, K, V, generator=gen) * 0.1
    do = torch.randn(B, L, Hv, V, generator=gen)
    dfs = torch.randn(B, Hv, K, V, generator=gen) * 0.1
    cu = lambda t: t.cuda()
    ins = [cu(t) for t in (q, k, v, g, b, w)]
    opts = dict(chunk_size=C, precision=prec, qk_l2norm=True)
    # (the hop-by-hop exchange on the configurations that recompute, the gathered one elsewhere)
    res = _run_sharded(n, ins, cu(seg), cu(init), cu(do), cu(dfs), exchange="p2p" if recompute else "gather",
                       recompute_states=recompute, **opts)

    # the unsharded operator on the same device
    leaves = [t.clone().requires_grad_() for t in ins]
    init_leaf = cu(init).requires_grad_()
    o1, f1 = dn.chunk_gdn2(*leaves, segment_ids=cu(seg), initial_state=init_leaf, output_final_state=True, **opts)
    g1 = torch.autograd.grad((o1.float() * cu(do)).sum() + (f1 * cu(dfs)).sum(), leaves + [init_leaf])
    out = torch.cat([r["out"] for r in res], 1)
    assert O.rel_l2(out.cpu(), o1.detach().cpu()) < tol
    assert O.rel_l2(res[-1]["final"].cpu(), f1.detach().cpu()) < tol
    for i in range(6):
        got = torch.cat([r["grads"][i] for r in res], 1)
        assert O.rel_l2(got.cpu(), g1[i].cpu()) < tol, i
    assert O.rel_l2(res[0]["grads"][6].cpu(), g1[6].cpu()) < tol

    # every rank's final_state is the state after its shard: rank 0's equals a call on the first shard alone
    _, f_first = dn.chunk_gdn2(*(t[:, :L // n].contiguous() for t in ins), segment_ids=cu(seg)[:, :L // n].contiguous(),
                               initial_state=cu(init), output_final_state=True, **opts)
    assert O.rel_l2(res[0]["final"].cpu(), f_first.cpu()) < tol

    # and the CPU oracle on the unsplit sequence (fp32 only: the bf16 pair above shares its rounding)
    if prec == "fp32":
        o_ref, f_ref = O.chunk_gdn2(q, k, v, g, b, w, segment_ids=seg, initial_state=init, output_final_state=True, **opts)
        assert O.rel_l2(out.cpu(), o_ref) < tol and O.rel_l2(res[-1]["final"].cpu(), f_ref) < tol


@pytest.mark.parametrize("n,prec,C,K,V,tol", [(2, "fp32", 64, 64, 64, 2e-4), (4, "bf16", 128, 128, 128, 2e-2)])
def test_sharded_without_initial_state_or_final_state_loss(n, prec, C, K, V, tol):
    """No initial state and no loss on the last final state: the first shard's forward correction and the
    last shard's backward correction are exact by construction and are skipped."""
    import deltanet_b200 as dn
    B, L, Hk, Hv = 1, 1024, 2, 4
    q, k, v, g, b, w = O.make_inputs(93, B, L, Hk, Hv, K, V, qkv_scale=0.5)
    seg = torch.repeat_interleave(torch.tensor([0, 1, 2], dtype=torch.int32), torch.tensor([200, 500, 324]))[None]
    do = torch.randn(B, L, Hv, V, generator=torch.Generator().manual_seed(6))
    cu = lambda t: t.cuda()
    ins = [cu(t) for t in (q, k, v, g, b, w)]
    opts = dict(chunk_size=C, precision=prec, qk_l2norm=True)
    res = _run_sharded(n, ins, cu(seg), None, cu(do), None, **opts)
    leaves = [t.clone().requires_grad_() for t in ins]
    o1, f1 = dn.chunk_gdn2(*leaves, segment_ids=cu(seg), output_final_state=True, **opts)
    g1 = torch.autograd.grad((o1.float() * cu(do)).sum(), leaves)
    assert O.rel_l2(torch.cat([r["out"] for r in res], 1).cpu(), o1.detach().cpu()) < tol
    assert O.rel_l2(res[-1]["final"].cpu(), f1.detach().cpu()) < tol
    for i in range(6):
        assert O.rel_l2(torch.cat([r["grads"][i] for r in res], 1).cpu(), g1[i].cpu()) < tol, i
