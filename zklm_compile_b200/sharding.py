"""Host-side logic for spreading independent per-layer proofs over several GPUs.

The reference proves the layers of a Qwen model with independent transcripts (seed
"qwen-layer-{idx}", rust/zk_ml_prover/src/pipeline/prove.rs:158-189) and collects the proofs in
reverse layer order (:183-188).  Here each rank owns a contiguous block of layers (4 per GPU
for 32 layers on 8 GPUs); only the d_model-word activation crosses from one rank to the next.
"""
from __future__ import annotations


def layer_range(rank: int, world: int, n_layers: int):
    """[lo, hi) of the layers owned by `rank`: contiguous blocks of ceil(n_layers / world)."""
    per = -(-n_layers // world)
    lo = min(rank * per, n_layers)
    return lo, min(lo + per, n_layers)


def owner_of(layer: int, world: int, n_layers: int) -> int:
    per = -(-n_layers // world)
    return layer // per


def merge_reverse(per_rank_proofs):
    """per_rank_proofs[r] = proofs of rank r's layers in reverse layer order (as QwenModel.prove
    returns them).  Result: all proofs in reverse global layer order."""
    return [p for chunk in reversed(per_rank_proofs) for p in chunk]


def send_activation(dist, tensor, dst: int):
    dist.send(tensor, dst=dst)


def recv_activation(dist, tensor, src: int):
    dist.recv(tensor, src=src)
