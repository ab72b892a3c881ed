"""The per-layer program: the fused call list (producer-side maxima, reduce-scatters pulled inside their consumers,
epoch bump inside the first barrier, routing tables inside the scatter launch) must leave exactly the bytes the
reference call list leaves -- flag counters and routing tables included -- for a KDA layer and an MLA layer, in
fewer launches."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "kern-k3_b200"))

pytestmark = pytest.mark.gpu

OUTPUTS = ["hidden", "normed_all", "fp8_big", "qscale", "prefix2_next", "normed", "fp8_small", "idx", "wts", "latent_q_all", "latent_sf_all", "wts_all",
           "idx_all", "route_map", "exp2perm", "moe_partial", "routed_latent_norm", "shared_act", "shared_q", "stats", "blocks",
           "blockoff", "cta_batch", "cta_limit", "nne", "total", "flags"]


@pytest.mark.parametrize("kind", ["kda", "mla"])
def test_fused_list_equals_reference_list(k3g, dev, kind):
    import torch
    from k3g.layer import LayerGlue
    got, launches = {}, {}
    for fused in (False, True):
        lg = LayerGlue(0, 1, tokens=1024, kind=kind, nb=3, seed=5, fused=fused)
        launches[fused] = lg.launches()
        lg.run()
        lg.run()                                  # a second pass: flags / epochs advance, results must not move
        torch.cuda.synchronize()
        lg.check_status()
        got[fused] = {name: getattr(lg, name).clone() for name in OUTPUTS}
        extra = ["span_q", "span_k", "span_v", "gated"] if kind == "kda" else ["q_norm", "mla_gate", "attn_gated", "latent_rows"]
        got[fused].update({name: getattr(lg, name).clone() for name in extra})
        lg.close()
    assert launches[True] < launches[False]
    bad = [name for name, ref in got[False].items() if not torch.equal(ref.view(torch.uint8), got[True][name].view(torch.uint8))]
    assert not bad, bad
