"""Token embeddings and the output head as parts.

Embedding: h[t, :] = E[id_t, :], no scaling (crates/ferrisinfer-kernel/src/cpu/attention.rs:3-99).
Output head: logits[v] = sum_k y[k] W[v, k], no bias, only for the rows asked
(crates/ferrisinfer-runtime/src/reference.rs:145-149); tied = the embedding table is W
(crates/ferrisinfer-runtime/src/reference.rs:976-982).
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, TensorSpec
from .plan import register_part


class TokenEmbedding(Part):
    def __init__(self, vocab_size: int, hidden_size: int, weight_name: str = "weight"):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.weight_name = weight_name  # "" = the tensor is named by the prefix itself
        self.weight = None

    def _name(self, prefix):
        return f"{prefix}.{self.weight_name}" if self.weight_name else prefix

    def tensor_specs(self, prefix):
        return [TensorSpec(self._name(prefix), (self.vocab_size, self.hidden_size), "embedding")]

    def bind(self, tensors, prefix):
        self.weight = tensors[self._name(prefix)]

    def forward(self, token_ids, h):
        ops.embed_gather(self.weight, token_ids, h)


class ScaledSinusoidalEmbedding(Part):
    """h[t, :] = E[id_t, :] * scale + pe(pos_t), with pe(p)[2i] = sin(p * base^(-2i / H)) and pe(p)[2i + 1] the cosine
    of the same angle.  The frequencies are formed in 64-bit on the host and rounded once; angles are fp32.
    ``needs_positions``: the model hands ``forward`` the step's positions.  ``base`` None: no position vector, the
    scaled table row alone (registered as ``scaled_embedding``)."""

    needs_positions = True

    def __init__(self, vocab_size: int, hidden_size: int, scale: float = 1.0, base: float = 10000.0,
                 weight_name: str = "weight"):
        self.vocab_size, self.hidden_size = int(vocab_size), int(hidden_size)
        self.scale, self.base, self.weight_name = float(scale), None if base is None else float(base), weight_name
        self.weight = None
        self._freq = {}

    def _name(self, prefix):
        return f"{prefix}.{self.weight_name}" if self.weight_name else prefix

    def tensor_specs(self, prefix):
        return [TensorSpec(self._name(prefix), (self.vocab_size, self.hidden_size), "embedding")]

    def bind(self, tensors, prefix):
        self.weight = tensors[self._name(prefix)]

    def frequencies(self, device) -> torch.Tensor:
        if self.base is None:
            return None
        key = str(device)
        if key not in self._freq:
            H = self.hidden_size
            f = [self.base ** (-2.0 * i / H) for i in range((H + 1) // 2)]
            self._freq[key] = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(device)
        return self._freq[key]

    def forward(self, token_ids, h, positions=None):
        ops.embed_sinusoid(self.weight, token_ids, positions, self.frequencies(h.device), self.scale, h)


class OutputHead(Part):
    """``tied_to``: tensor name of the embedding table to use as the output matrix, or None
    when the folder has a matrix of its own under ``prefix``.  ``softcap``: the logits z become
    softcap * tanh(z / softcap) (None: they stay as they are).  ``logit_scale``: a factor on the logits (before a cap)."""

    def __init__(self, vocab_size: int, hidden_size: int, tied_to=None, weight_name: str = "weight",
                 softcap: float = None, logit_scale: float = 1.0):
        self.vocab_size, self.hidden_size, self.tied_to = int(vocab_size), int(hidden_size), tied_to
        self.softcap = None if not softcap else float(softcap)
        if self.softcap is not None and not (self.softcap > 0.0):
            raise ValueError(f"a soft cap of {softcap}: a positive number is needed")
        self.logit_scale = float(logit_scale)
        self.weight_name = weight_name  # "" = the tensor is named by the prefix itself
        self.weight = None

    def _name(self, prefix):
        return f"{prefix}.{self.weight_name}" if self.weight_name else prefix

    def tensor_specs(self, prefix):
        if self.tied_to:
            return []
        return [TensorSpec(self._name(prefix), (self.vocab_size, self.hidden_size), "matrix")]

    def bind(self, tensors, prefix):
        self.weight = tensors[self.tied_to if self.tied_to else self._name(prefix)]

    def forward(self, y, logits):
        """logits fp32 [n, V] = y [n, H] W^T."""
        ops.gemm(y, self.weight, None, logits)
        if self.logit_scale != 1.0:
            ops.scale_(logits, self.logit_scale)
        if self.softcap is not None:
            ops.softcap_(logits, self.softcap)

    def forward_greedy(self, y, tokens, probs, workspace):
        """tokens int32 [n] = the index of each row's greatest logit (the lowest among equals), probs fp32 [n] its
        softmax probability; the logits themselves are stored nowhere where a kernel can avoid it (the reference's
        fused product + argmax: crates/ferrisinfer-kernel/src/cpu/matmul.rs:190-274)."""
        if self.softcap is not None or self.logit_scale != 1.0:
            # a cap or a factor changes the probabilities (a negative factor also the order): logits, factor, cap, then
            # the greedy rows
            logits = workspace.get("logits", (y.shape[0], self.vocab_size), torch.float32)
            self.forward(y, logits)
            ops.sample(logits, tokens, probs)
            return
        ops.greedy_head(y, self.weight, tokens, probs, workspace)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "scaled_sinusoidal_embedding", ScaledSinusoidalEmbedding)
register_part("embedding", "scaled_embedding",
              lambda vocab_size, hidden_size, scale=1.0, weight_name="weight": ScaledSinusoidalEmbedding(
                  vocab_size, hidden_size, scale=scale, base=None, weight_name=weight_name))
register_part("output", "linear_head", OutputHead)
