"""The decode layer under its launch modes (environment switch read once per process, hence child processes): the
single kernel launched automatically (default: programmatic stream serialisation for the first stream of a device,
cooperative for any other), programmatically for every stream, cooperatively for every stream, and the two-kernel
chain.  Each child checks the layer against the CPU oracle and against a repeat call (bitwise)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import importlib, sys
import numpy as np, torch
sys.path.insert(0, {root!r})
import __graft_entry__ as entry
import oracle
entry.load_package()
gb = importlib.import_module("dsv4_b200.runtime.mxfp4_grouped_gemv_binding")
qz = importlib.import_module("dsv4_b200.runtime.quantize")
dev = torch.device("cuda:0")
E, K, H, k = 16, 4096, 2048, 6
bank = qz.make_expert_bank(E, K, H, "cpu", seed=11)
dbank = {{n: v.to(dev) for n, v in bank.items()}}
g = torch.Generator().manual_seed(5)
worst = 0.0
for step in range(6):                      # several layers back to back
    x = torch.randn(K, generator=g).to(torch.bfloat16)
    logits = torch.randn(E, generator=g)
    out = gb.moe_decode_layer(dbank, logits.to(dev), x.to(dev), k=k, score_func="softmax")
    again = gb.moe_decode_layer(dbank, logits.to(dev), x.to(dev), k=k, score_func="softmax")
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))
    ids, w = oracle.route_softmax(logits.numpy()[None], k)
    ref = oracle.moe_layer_ref(x[None], bank, ids, w)[0]
    got = out.float().cpu().numpy()
    err, cos = oracle.max_abs_rel(got, ref), oracle.cosine(got, ref)
    assert err <= 5e-3 and cos >= 0.99999, (step, err, cos)
    worst = max(worst, err)
assert gb.device_status() == 0
print("ok", worst)
"""


@pytest.mark.parametrize("mode", ["auto", "coop", "pdl", "0"])
def test_decode_layer_launch_modes(mode):
    env = dict(os.environ, DSV4_B200_FUSED=mode)
    r = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT)], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.strip().splitlines()[-1].startswith("ok")
