"""Whole-network INT8 ResNet-50 (BASELINE config 3 at a small batch): executor vs the oracle, every tensor bit exact."""
import numpy as np
import pytest
import torch

import oracle_graph
from tpu_mlir_b200 import resnet50, synth
from tpu_mlir_b200.module import module

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lowered():
    ops = resnet50.build_fp32(seed=3)
    images = torch.from_numpy(synth.calibration_images(seed=4, count=8)).cuda()
    table = resnet50.self_calibration_table(ops, images, batch=4)
    graph, weights = resnet50.lower_int8(ops, table, batch=2)
    return ops, table, graph, weights


@pytest.mark.parametrize("channels_last", [False, True])
def test_int8_graph_matches_oracle_on_every_tensor(lowered, channels_last):
    ops, table, graph, weights = lowered
    x = synth.calibration_images(seed=33, count=2)
    m = module(channels_last=channels_last)
    m.load(graph, weights)
    seen = []
    m.after_invoke(lambda name: seen.append(name))
    m.set_tensor("input", x)
    m.invoke(fixed_to_float=False)
    assert seen == [op["name"] for op in graph["ops"]]
    if channels_last:   # every activation between the stem and the classifier lives as [N][H][W][C]
        assert len(m._nhwc) > 60 and tuple(m.tensors["conv1"].shape) == (2, 112, 112, 64)
    want = oracle_graph.run(graph, weights, {"input": x})
    types = {}
    for op in graph["ops"]:
        name = op["name"]
        got = m.get_tensor(name)
        assert np.array_equal(got, want[name]), (name, op["type"])
        types[graph["tensors"][name]["dtype"]] = types.get(graph["tensors"][name]["dtype"], 0) + 1
    assert types.get("u8", 0) > 40 and types.get("i8", 0) > 10      # post-ReLU tensors are unsigned
    logits = m.get_tensor("fc")
    assert logits.shape == (2, 1000) and logits.dtype == np.int8 and len(np.unique(logits)) > 20
    # the expressed (float) view of a quantized tensor
    info = graph["tensors"]["fc"]
    assert np.allclose(m.get_fp32_tensor("fc"), logits.astype(np.float32) * np.float32(info["scale"]))


def test_cuda_graph_replay_matches_eager(lowered):
    ops, table, graph, weights = lowered
    eager = module(channels_last=True)
    eager.load(graph, weights)
    fast = module(channels_last=True, cuda_graph=True)
    fast.load(graph, weights)
    for seed in (35, 36):       # the second input goes through the replay of the graph captured for the first
        x = synth.calibration_images(seed=seed, count=2)
        for m in (eager, fast):
            m.set_tensor("input", x)
            m.invoke(fixed_to_float=False)
        for name in ("conv1", "layer2.0.add", "layer4.2.conv3", "fc", "output"):
            assert np.array_equal(eager.get_tensor(name), fast.get_tensor(name)), (seed, name)
    assert fast._graph is not None
    seen = []
    fast.after_invoke(lambda name: seen.append(name))      # hooks need the op-by-op path
    fast.invoke(fixed_to_float=False)
    assert len(seen) == len(graph["ops"])


def test_int8_logits_track_the_fp32_network(lowered):
    ops, table, graph, weights = lowered
    x = synth.calibration_images(seed=34, count=2)
    m = module()
    m.load(graph, weights)
    m.set_tensor("input", x)
    m.invoke(fixed_to_float=False)
    q = m.get_tensor("output")
    f = resnet50.Fp32Forward(ops, torch.device("cuda"))(torch.from_numpy(x).cuda())["fc"].cpu().numpy()
    cos = float((q * f).sum() / (np.linalg.norm(q) * np.linalg.norm(f)))
    assert cos > 0.95, cos          # the reference's own int8-vs-fp32 acceptance level (test_onnx.py:624-640)


def test_fused_residual_adds_keep_every_other_tensor(lowered):
    """module(fuse_residual_add=True): the 16 residual Adds run inside the kernels of the convolutions that feed them;
    every tensor that is still materialised equals the oracle's, the fused-away convolution outputs raise."""
    ops, table, graph, weights = lowered
    x = synth.calibration_images(seed=37, count=2)
    m = module(channels_last=True, cuda_graph=True, fuse_residual_add=True)
    m.load(graph, weights)
    assert len(m._fused_adds) == 16
    m.set_tensor("input", x)
    m.invoke(fixed_to_float=False)
    want = oracle_graph.run(graph, weights, {"input": x})
    for op in graph["ops"]:
        name = op["name"]
        if name in m._fuse_into:
            with pytest.raises(Exception):
                m.get_tensor(name)
            continue
        assert np.array_equal(m.get_tensor(name), want[name]), (name, op["type"])
    # one op at a time: a fused Add is produced by running its convolution
    add = next(iter(m._fused_adds))
    assert np.array_equal(m.invoke_at(add), want[add])
