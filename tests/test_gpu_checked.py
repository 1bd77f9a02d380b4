"""Index checks on plan contents: a corrupt or foreign plan must end in a recorded status
(``MoonEPTimeout`` with the "index out of range" code), never in an access outside the buffers.

Always on: destination ranks named by ``plan.dst`` (dispatch, combine) and a token without any
primary row (combine).  With ``MOONEP_CHECKED=1`` the duplicate-row kernels additionally report
table entries they would otherwise skip silently.  Poisoned shards and sentinel-wrapped outputs
prove that nothing outside the valid targets was written.
"""
import numpy as np
import pytest
import torch

from moonep_b200 import engine
from moonep_b200.plan import MoonEPCommPlan
from moonep_b200.sim.local_cluster import LocalCluster

from gpu_helpers import make_topk, traceable_hidden

pytestmark = pytest.mark.gpu


def _fresh(R=2, S=64, K=4, epn=4, H=256, pad=16, **kw):
    E = R * epn
    topk, tpe = make_topk("random", S, K, E, R, seed=5)
    cl = LocalCluster(S, H, K, E, R, num_sms=2, token_padding=pad, budget_ms=200, **kw)
    dev = cl.device
    hidden = [traceable_hidden(S, H, r).to(dev) for r in range(R)]
    oh, _, cus, plans = cl.dispatch(hidden, None, [t.to(dev) for t in topk], [t.to(dev) for t in tpe])
    torch.cuda.synchronize()
    cl.check()
    return cl, plans, hidden


def _with(plan: MoonEPCommPlan, **repl) -> MoonEPCommPlan:
    kw = {f: getattr(plan, f) for f in plan.__dataclass_fields__}
    kw.update(repl)
    return MoonEPCommPlan(**kw)


def test_dispatch_reports_a_destination_outside_the_group(cuda_device):
    cl, plans, hidden = _fresh()
    g = cl.geo
    bad = plans[0].dst.clone()
    bad[5] = g.R * g.NvS + 3            # rank R does not exist
    bad[9] = -(g.R * g.NvS + 7) - 1     # same, encoded as a duplicate
    for s in cl._states:
        s.hidden_local.view(torch.int16).fill_(0x5555)
    before = cl.heap.whole().clone()
    cl.dispatch(hidden, None, plans=[_with(plans[0], dst=bad), plans[1]])
    torch.cuda.synchronize()
    with pytest.raises(engine.MoonEPTimeout) as ei:
        cl.check()
    assert ei.value.status["code"] == 3 and ei.value.status["kernel"] == 3
    # the bad entries wrote nothing: every byte that changed lies inside a hidden shard or is a barrier word
    after = cl.heap.whole()
    changed = (after != before).nonzero().flatten().cpu().numpy()
    off = changed % cl.heap.chunk_bytes
    in_hidden = (off >= g.off_hidden) & (off < g.off_hidden + g.NvS * g.H * 2)
    in_barrier = (off >= g.off_bar) & (off < g.off_bar + 4 * 128 * 4)
    assert np.all(in_hidden | in_barrier)


def test_combine_reports_bad_destinations_and_tokens_without_rows(cuda_device):
    cl, plans, hidden = _fresh()
    g = cl.geo
    bad = plans[1].dst.clone()
    bad[0:g.K] = -(g.R * g.NvS) - 1     # token 0: every entry a duplicate on a rank that does not exist
    outs, _ = cl.combine([plans[0], _with(plans[1], dst=bad)], [s.hidden_local for s in cl._states], zero_copy=True)
    torch.cuda.synchronize()
    with pytest.raises(engine.MoonEPTimeout) as ei:
        cl.check()
    assert ei.value.status["code"] == 3 and ei.value.status["kernel"] == 6
    assert torch.count_nonzero(outs[1][0]) == 0            # the row-less token comes back as zeros


def test_checked_mode_reports_corrupt_duplicate_tables(cuda_device, monkeypatch):
    monkeypatch.setenv("MOONEP_CHECKED", "1")
    cl, plans, hidden = _fresh()
    g = cl.geo
    assert cl._states[0].ctx_host.checked == 1
    n = int(plans[0].dup_counts[0])
    assert n > 0, "the routing must produce duplicate rows"
    groups = plans[0].dup_groups.clone()
    groups[0, 0] = g.NvS + 11           # primary row outside the shard
    from moonep_b200 import engine as eng
    eng.launch_dup_expand(cl._states, [s.hidden_local for s in cl._states], [_with(plans[0], dup_groups=groups), plans[1]], 8)
    torch.cuda.synchronize()
    with pytest.raises(engine.MoonEPTimeout) as ei:
        cl.check()
    assert ei.value.status["code"] == 3 and ei.value.status["kernel"] == 4


def test_unchecked_mode_skips_corrupt_duplicate_tables_quietly(cuda_device, monkeypatch):
    monkeypatch.delenv("MOONEP_CHECKED", raising=False)
    cl, plans, hidden = _fresh()
    g = cl.geo
    groups = plans[0].dup_groups.clone()
    groups[0, 0] = g.NvS + 11
    engine.launch_dup_expand(cl._states, [s.hidden_local for s in cl._states], [_with(plans[0], dup_groups=groups), plans[1]], 8)
    torch.cuda.synchronize()
    cl.check()
