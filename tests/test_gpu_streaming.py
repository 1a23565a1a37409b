"""Host-to-host streaming through a layer: batches queued back to back on three streams must
come back in order and equal to what the layer gives for each batch alone."""
import pytest
import torch

from gpu_util import rel_fro, seeded

pytestmark = pytest.mark.gpu


def test_streamed_batches_match_direct_calls():
    from lcgemm import ops
    from lcgemm.layer import Rank7MlpLayer
    from lcgemm.streaming import HostStreamedLayer

    m, h, i = 512, 256, 1024
    nw, wgu, wd = seeded((h,), 3, 0.01), seeded((2 * i, h), 4, 0.02), seeded((h, i), 5, 0.02)
    layer = Rank7MlpLayer(m, nw, wgu, wd)
    batches = [seeded((m, h), 50 + b, device="cpu").pin_memory() for b in range(7)]
    want = [layer(b.cuda()).clone() for b in batches]
    outs = [torch.zeros((m, h), dtype=torch.bfloat16).pin_memory() for _ in batches]
    st = HostStreamedLayer(layer, m, h)
    st.begin()
    for b, o in zip(batches, outs):
        st.submit(b, o)
    st.end()
    st.drain()
    ops.check_status()
    for b in range(len(batches)):
        assert rel_fro(outs[b], want[b]) <= 8e-3, b               # unordered bf16 adds of the split tail
        if b:
            assert rel_fro(outs[b], want[b - 1]) > 0.5            # and not some other batch's result
    # a second run over the same streamer reuses the buffers
    st.begin()
    st.submit(batches[2], outs[0])
    st.end()
    st.drain()
    assert rel_fro(outs[0], want[2]) <= 8e-3


def test_captured_layer_replays_the_same_kernels():
    from lcgemm import ops
    from lcgemm.layer import CapturedLayer, DenseMlpLayer, Rank7MlpLayer

    m, h, i = 512, 256, 1024
    nw, wgu, wd = seeded((h,), 3, 0.01), seeded((2 * i, h), 4, 0.02), seeded((h, i), 5, 0.02)
    x = seeded((m, h), 60)
    for layer in (Rank7MlpLayer(m, nw, wgu, wd), DenseMlpLayer(m, nw, wgu, wd)):
        want = layer(x).clone()
        before = ops.launch_count()
        graph = CapturedLayer(layer, x)
        recorded = ops.launch_count() - before          # warm-up calls + the recorded one
        for _ in range(3):
            got = graph()
        assert ops.launch_count() - before == recorded  # replays go through no host-side launch
        assert rel_fro(got, want) <= 8e-3
        x2 = seeded((m, h), 61)
        want2 = layer(x2).clone()
        x.copy_(x2)                                      # the recording reads x's storage
        assert rel_fro(graph(), want2) <= 8e-3
        x.copy_(seeded((m, h), 60))
    ops.check_status()
