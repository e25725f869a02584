"""The benchmark networks (cfg3, cfg5) on the CUDA operators vs the same networks on the CPU oracle:
loss and every parameter gradient of one forward + backward step, at a small batch."""
import numpy as np
import pytest
import torch

import cases
from simnets_tf_b200 import dp
from simnets_tf_b200.simnet import SPECS, SimNet

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,batch", [("cfg3", 6), ("cfg5", 4)])
def test_network_step_matches_cpu_oracle(port, name, batch):
    from oracle.simnet_cpu import CpuSimNet
    spec = SPECS[name]
    rng = np.random.default_rng(11)
    x = rng.uniform(-0.5, 0.5, size=(batch,) + tuple(spec["input_shape"])).astype(np.float32)
    labels = rng.integers(0, spec["classes"], size=batch)
    cpu = CpuSimNet(spec, port, seed=5, threads=2)
    ref_loss, ref_grads = cpu.step(x, labels)
    net = SimNet(spec, seed=5, device="cuda")
    bucket = dp.GradBucket(net.parameters())
    bucket.zero()
    loss = net.loss(torch.from_numpy(x).cuda(), torch.from_numpy(labels).cuda())
    loss.backward()
    assert abs(float(loss) - ref_loss) <= 1e-5 * abs(ref_loss)
    params = list(net.parameters())
    assert len(params) == len(ref_grads)
    assert sum(p.numel() for p in params) == {"cfg3": 701696, "cfg5": 773504}[name]
    for i, (p, g) in enumerate(zip(params, ref_grads)):
        assert p.grad.data_ptr() >= bucket.flat.data_ptr()          # gradients live inside the flat bucket
        cases.assert_parity(p.grad.cpu().numpy(), g, tol=5e-5, what="%s grad %d %s" % (name, i, tuple(p.shape)))
