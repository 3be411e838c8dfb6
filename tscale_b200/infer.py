"""Host-side mirror of the reference's KV-cache inference (NCPUInfer, code/gpt/train/cpu_infer.cpp:466-560) over
tsa_infer_step: `InferModel` holds the int8 model on the device (TCPUModelParams), `InferContext` the per-layer KV
caches of a batch of sequences (TCPUInferContext), `compute_prediction` is ComputePrediction for the whole batch.
No computation happens here: every step is one call into the shared library."""
import ctypes

import numpy as np
import torch

from . import abi
from .abi import check
from .ops import _ptr, _stream

_MATS = ("qk", "qv", "k", "v", "combiner", "expand", "contract")


class InferModel:
    """model: dict as oracle.make_infer_model builds it (numpy int8 matrices and float scales), copied to `device`.
    rope: float32 [rope_len][head_dim] table (FillRopeBuf, code/gpt/att/rope.cpp:4-24); positions beyond it are an error."""

    def __init__(self, model, rope, device):
        self.device = device
        self.dim, self.head_dim, self.heads = model["dim"], model["head_dim"], model["heads"]
        self.relu_dim = self.heads * 128 * model["relu_mult"]
        self.vocab, self.label_count = model["vocab"], model["label_count"]
        self._keep = []

        def dev(a, dtype):
            t = torch.from_numpy(np.ascontiguousarray(a)).to(device=device, dtype=dtype)
            self._keep.append(t)
            return t

        n = len(model["layers"])
        self._layers = (abi.InferLayer * max(n, 1))()
        for i, layer in enumerate(model["layers"]):
            rec = self._layers[i]
            for nm in _MATS:
                setattr(rec, nm, dev(layer[nm], torch.int8).data_ptr())
            rec.qv_scale, rec.combiner_scale, rec.contract_scale = float(layer["qv_scale"]), float(layer["combiner_scale"]), float(layer["contract_scale"])
            rec.attention_width, rec.alibi_slope = int(layer["width"]), float(layer["slope"])
        self.rope = dev(rope, torch.float32)
        self.c = abi.InferModel()
        self.c.dims = abi.InferDims(self.dim, self.head_dim, self.heads, self.relu_dim, self.vocab, self.label_count, n)
        self.c.layers = ctypes.cast(self._layers, ctypes.POINTER(abi.InferLayer))
        self.c.label_embed = dev(model["label_embed"], torch.int8).data_ptr()
        self.c.label_embed_scale = float(model["label_embed_scale"])
        self.c.final_layer = dev(model["final_layer"], torch.int8).data_ptr()
        self.c.final_layer_scale = float(model["final_layer_scale"])
        self.c.bias = dev(model["bias"], torch.float32).data_ptr()
        self.c.rope = self.rope.data_ptr()
        self.c.rope_len = int(self.rope.shape[0])
        self.layer_count = n


class InferContext:
    """KV caches of n_seq sequences for every layer (int8 keys and values, f32 scale planes), `capacity` tokens each."""

    def __init__(self, model, n_seq, capacity):
        self.model, self.n_seq, self.capacity = model, n_seq, capacity
        dev, row, heads, n = model.device, model.heads * model.head_dim, model.heads, model.layer_count
        self.k = torch.zeros((n, n_seq, capacity, row), dtype=torch.int8, device=dev)
        self.v = torch.zeros((n, n_seq, capacity, row), dtype=torch.int8, device=dev)
        self.k_scale = torch.zeros((n, n_seq, capacity, heads), dtype=torch.float32, device=dev)
        self.v_scale = torch.zeros((n, n_seq, capacity, heads), dtype=torch.float32, device=dev)
        self.ctx_lens = torch.zeros((max(n, 1), n_seq), dtype=torch.int32, device=dev)
        table = np.zeros((max(n, 1), n_seq, 4), dtype=np.uint64)
        for l in range(n):
            for s in range(n_seq):
                table[l, s] = (self.k[l, s].data_ptr(), self.v[l, s].data_ptr(), self.k_scale[l, s].data_ptr(), self.v_scale[l, s].data_ptr())
        self.seqs = torch.from_numpy(table.view(np.int64)).to(dev)
        self.layer_seqs = (ctypes.c_void_p * max(n, 1))(*[self.seqs[l].data_ptr() for l in range(max(n, 1))])
        self.max_ctx = 0
        need = abi.lib().tsa_infer_workspace_bytes(ctypes.byref(model.c), n_seq, capacity - 1)
        self.workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)

    def set_lengths(self, lens):
        """Declares that the caches already hold lens[s] tokens per sequence (bench set-up with pre-filled caches)."""
        t = torch.tensor(lens, dtype=torch.int32, device=self.model.device)
        self.ctx_lens.copy_(t.unsqueeze(0).expand_as(self.ctx_lens))
        self.max_ctx = int(max(lens))

    def compute_prediction(self, labels, prediction=None, logits=None, want_prediction=True, max_ctx_bound=None):
        """One token per sequence.  labels: int32 device tensor [n_seq][labels per token].  Returns the distribution
        over the vocabulary [n_seq][vocab] (None with want_prediction=False: the caches advance all the same).
        max_ctx_bound: upper bound of the token counts to size the launches for instead of the tracked maximum; a
        step captured into a CUDA graph and replayed many times needs the bound of its last replay."""
        m = self.model
        assert labels.dtype == torch.int32 and labels.dim() == 2 and labels.shape[0] == self.n_seq and labels.is_contiguous()
        if want_prediction and prediction is None:
            prediction = torch.empty((self.n_seq, m.vocab), dtype=torch.float32, device=m.device)
        check(abi.lib().tsa_infer_step(ctypes.byref(m.c), self.layer_seqs, _ptr(self.ctx_lens), self.capacity, _ptr(labels), labels.shape[1],
                                       self.n_seq, self.max_ctx if max_ctx_bound is None else int(max_ctx_bound), _ptr(prediction), _ptr(logits), _ptr(self.workspace), self.workspace.numel(),
                                       _ptr(self.status), _stream()))
        self.max_ctx += 1
        return prediction
