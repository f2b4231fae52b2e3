"""Host I/O path (tagi_io_*): batches staged in pinned memory, uploaded on the pipeline's own stream, exactly B x n_out
output moments read back. A small MLP trained through the pipeline must behave bit for bit like the same network fed by
plain copies; slot reuse is ordered by the consumed / uploaded events, so two slots may be in flight."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _net(seed):
    from cutagi_b200 import nn
    return nn.Sequential(nn.Linear(24, 64, seed=seed), nn.ReLU(), nn.Linear(64, 11, seed=seed + 1))


def test_training_through_the_pipeline_matches_plain_copies():
    import torch
    from cutagi_b200 import nn
    from cutagi_b200.hostio import HostPipeline
    B, steps = 16, 6
    rng = np.random.default_rng(0)
    xs = rng.standard_normal((steps, B, 24)).astype(np.float32)
    utils = nn.Utils()
    lab = [utils.label_to_obs(rng.integers(0, 10, B), 10) for _ in range(steps)]
    var_y = torch.full((B * 4,), 1.0, device="cuda")
    ref, upd = _net(5), nn.OutputUpdater()
    want = []
    for s in range(steps):
        mu, var = ref(xs[s])
        want.append((mu.cpu().numpy().copy(), var.cpu().numpy().copy()))
        upd.update_using_indices(ref, lab[s][0], var_y, lab[s][1])
        ref.backward()
        ref.step()
    net = _net(5)
    io = HostPipeline(B * 24, B * 4, B * 4, B * 11, depth=2)
    sp = torch.cuda.current_stream().cuda_stream
    try:
        def stage(s):
            x, obs, idx = io.host_arrays(s % 2)
            x[:], obs[:], idx[:] = xs[s].reshape(-1), lab[s][0], lab[s][1]
        stage(0)
        for s in range(steps):
            slot = s % 2
            mu, var, obs, idx = net.forward_staged(io, slot)
            if s + 1 < steps:
                stage(s + 1)     # the host fills the other slot while the device works on this one
            upd.update_using_indices(net, obs, var_y, idx)
            net.backward()
            net.step()
            io.consumed(slot, sp)
            io.download(slot, mu, var, sp)
            hm, hv = io.wait_output(slot, B * 11)
            assert np.array_equal(hm.reshape(B, 11), want[s][0]) and np.array_equal(hv.reshape(B, 11), want[s][1]), s
        net.check_kernels()
    finally:
        io.close()


def test_argument_errors():
    import torch
    from cutagi_b200.capi import TagiError
    from cutagi_b200.hostio import HostPipeline
    with pytest.raises(TagiError):
        HostPipeline(16, 0, 0, 8, depth=0)
    io = HostPipeline(16, 4, 4, 8, depth=2)
    try:
        t = torch.zeros(16, device="cuda")
        sp = torch.cuda.current_stream().cuda_stream
        with pytest.raises(TagiError) as e:
            io.download(0, t, t, sp)             # 16 floats into a pipeline sized for 8
        assert "capacity" in str(e.value)
        with pytest.raises(TagiError):
            io.upload(2, sp)                     # slot out of range
    finally:
        io.close()
