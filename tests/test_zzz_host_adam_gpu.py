"""Optimizer state resident in pinned host memory (``swap_optimizer``): streaming it through the GPU in chunks
on copy streams gives the same parameters as keeping it on the device."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(offload: bool, dtype):
    from mindspeed_rl_b200.optim.distributed_optimizer import DistributedOptimizer
    from mindspeed_rl_b200.parallel.ddp import DistributedDataParallel
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(512, 1024), torch.nn.Linear(1024, 384)).to("cuda", dtype)
    ddp = DistributedDataParallel(net, None, 1)
    opt = DistributedOptimizer(ddp.buffers, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.01, clip_grad=1.0,
                               offload_to_host=offload, swap_chunks=7)
    return net, ddp, opt


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_host_resident_state_matches_device_resident(dtype):
    nets = [_build(False, dtype), _build(True, dtype)]
    assert all(t.is_pinned() for t in nets[1][2].state[0].values())
    for step in range(3):
        g = torch.Generator(device="cuda").manual_seed(step)
        for net, ddp, opt in nets:
            ddp.zero_grad_buffer()
            for p in net.parameters():
                p.main_grad.copy_(0.05 * torch.randn(p.shape, device="cuda", generator=g.manual_seed(step)))
            ddp.finish_grad_sync(to_shards=True)
            opt.step()
    torch.cuda.synchronize()
    for a, b in zip(nets[0][0].parameters(), nets[1][0].parameters()):
        assert torch.allclose(a.float(), b.float(), atol=1e-6, rtol=0), float((a.float() - b.float()).abs().max())
    dev_state, host_state = nets[0][2].state[0], nets[1][2].state[0]
    for k in ("master", "exp_avg", "exp_avg_sq"):
        assert torch.allclose(dev_state[k].cpu(), host_state[k], atol=1e-7, rtol=1e-6), k
    sd = nets[1][2].state_dict()
    assert sd["step"] == 3 and torch.equal(sd["shards"][0]["master"], host_state["master"])
