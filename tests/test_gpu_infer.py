"""tsa_infer_step (one token per sequence through the int8 model with KV caches) against the oracle's restatement of
NCPUInfer::ComputePrediction and against the reference's own predictions (tests/golden/infer_*.npz)."""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.util import INFER_CASES

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _run_gpu(model, labels, capacity=None, want_logits=False):
    """labels int32 [n_seq][steps][labels per token] -> predictions [n_seq][steps][vocab] (and logits)."""
    from tscale_b200 import infer
    n_seq, steps = labels.shape[:2]
    rope = O.fill_rope(model["head_dim"], steps)
    gm = infer.InferModel(model, rope, DEV)
    ctx = infer.InferContext(gm, n_seq, capacity or steps)
    pred = np.zeros((n_seq, steps, model["vocab"]), dtype=np.float32)
    logits = np.zeros_like(pred)
    lg = torch.empty((n_seq, model["vocab"]), dtype=torch.float32, device=DEV) if want_logits else None
    for t in range(steps):
        lab = torch.from_numpy(np.ascontiguousarray(labels[:, t])).to(DEV)
        p = ctx.compute_prediction(lab, logits=lg)
        pred[:, t] = p.cpu().numpy()
        if want_logits:
            logits[:, t] = lg.cpu().numpy()
    torch.cuda.synchronize()
    assert int(ctx.status.item()) == 0
    assert ctx.ctx_lens.cpu().numpy().tolist() == [[steps] * n_seq] * max(len(model["layers"]), 1)
    return (pred, logits) if want_logits else pred


def _deviation(got, want):
    return np.abs(got - want).max(axis=-1) / want.max(axis=-1)


@pytest.mark.parametrize("name", ["infer_d64", "infer_d128"])
def test_against_reference_fixture(golden_dir, name):
    """The reference's predictions: its polynomial 2^x against exp2 here moves attention weights by 1e-4, and a
    flipped int8 rounding of a combiner input shows as up to 2 % of the largest probability in these small models."""
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    model = O.make_infer_model(**INFER_CASES[name])
    pred = _run_gpu(model, z["labels"])
    dev = _deviation(pred, z["prediction"])
    assert dev.max() < 5e-2 and np.median(dev) < 2e-3, (dev.max(), np.median(dev))
    assert np.abs(pred.sum(axis=-1) - 1).max() < 1e-5


@pytest.mark.parametrize("name", ["infer_d64", "infer_d128"])
def test_against_oracle_exact_exp(golden_dir, name):
    """Against the oracle with exact exp2: only the order of the attention sums and the 16-bit weights of the decode
    kernel differ, so nearly every step agrees to float rounding."""
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    model = O.make_infer_model(**INFER_CASES[name])
    pred = _run_gpu(model, z["labels"])
    n_seq, steps = z["labels"].shape[:2]
    want = np.zeros_like(pred)
    for s in range(n_seq):
        orc = O.InferOracle(model, steps, exp_mode="exact")
        for t in range(steps):
            want[s, t] = orc.step(z["labels"][s, t])
    dev = _deviation(pred, want)
    assert dev.max() < 5e-2 and np.median(dev) < 1e-4, (dev.max(), np.median(dev))


def test_first_step_bit_exact_and_batch_independence():
    """With windows > 0 the first token attends nothing, so every stage is integer or single-rounded float
    arithmetic: the final layer's int32 products must equal the oracle's exactly.  Sequences of a batch are
    independent: the same label stream gives the same bits in any slot and any batch size (33 > one lane group)."""
    model = O.make_infer_model(90, 512, 64, 4, 1, 1000, 64, [(16, 0.5), (128, 0.0)])
    rng = np.random.default_rng(91)
    steps = 6
    streams = rng.integers(0, 64, (3, steps, 2)).astype(np.int32)
    labels = np.concatenate([streams, streams[rng.integers(0, 3, 30)]], axis=0)   # 33 sequences
    pred, logits = _run_gpu(model, labels, want_logits=True)
    for s in range(3):
        orc = O.InferOracle(model, steps, exp_mode="exact")
        _, want_logits = orc.step(streams[s, 0], want_logits=True)
        assert np.array_equal(logits[s, 0], want_logits), s
    for s in range(3, 33):
        src = next(i for i in range(3) if np.array_equal(labels[s], streams[i]))
        assert np.array_equal(pred[s], pred[src]) and np.array_equal(logits[s], logits[src]), s
    alone = _run_gpu(model, streams[1:2])
    assert np.array_equal(alone[0], pred[1])


def test_wide_matrices_chunked_through_shared_memory():
    """64 sequences with a combiner input of 4 * 1536 columns: the batch's vectors do not fit shared memory at once."""
    model = O.make_infer_model(92, 256, 128, 12, 1, 64, 16, [(8, 0.0)])
    rng = np.random.default_rng(93)
    steps = 3
    streams = rng.integers(0, 16, (2, steps, 1)).astype(np.int32)
    labels = np.concatenate([streams] * 32, axis=0)   # 64 sequences
    pred, logits = _run_gpu(model, labels, want_logits=True)
    for s in range(2):
        orc = O.InferOracle(model, steps, exp_mode="exact")
        _, want_logits = orc.step(streams[s, 0], want_logits=True)
        assert np.array_equal(logits[s, 0], want_logits), s
    for s in range(2, 64):
        assert np.array_equal(logits[s], logits[s % 2]), s


def test_bad_arguments():
    from tscale_b200 import abi, infer
    model = O.make_infer_model(94, 256, 64, 2, 1, 32, 8, [(8, 0.0)])
    gm = infer.InferModel(model, O.fill_rope(64, 4), DEV)
    ctx = infer.InferContext(gm, 2, 4)
    lab = torch.zeros((2, 1), dtype=torch.int32, device=DEV)
    for _ in range(4):
        ctx.compute_prediction(lab)
    with pytest.raises(abi.TsaError):          # cache and rope table are full
        ctx.compute_prediction(lab)
    ctx2 = infer.InferContext(gm, 2, 4)
    bad = torch.full((2, 1), 99, dtype=torch.int32, device=DEV)   # label outside the embedding table
    ctx2.compute_prediction(bad)
    torch.cuda.synchronize()
    assert int(ctx2.status.item()) != 0


def test_batch_of_twenty_sequences():
    """17 to 32 sequences take the matrix products' two-way sequence split: exact first-step logits, identical slots."""
    model = O.make_infer_model(95, 256, 64, 2, 1, 96, 16, [(8, 0.0), (32, 0.5)])
    rng = np.random.default_rng(96)
    steps = 4
    streams = rng.integers(0, 16, (2, steps, 1)).astype(np.int32)
    labels = np.concatenate([streams] * 10, axis=0)   # 20 sequences
    pred, logits = _run_gpu(model, labels, want_logits=True)
    for s in range(2):
        orc = O.InferOracle(model, steps, exp_mode="exact")
        _, want_logits = orc.step(streams[s, 0], want_logits=True)
        assert np.array_equal(logits[s, 0], want_logits), s
    for s in range(2, 20):
        assert np.array_equal(logits[s], logits[s % 2]) and np.array_equal(pred[s], pred[s % 2]), s
