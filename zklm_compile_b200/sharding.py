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


# ---- gathering the proofs without pickling: one fixed-size byte tensor per rank ------------------
def pack_proofs(proofs, buf):
    """Writes [count u32][len u32 ...][bytes ...] into the 1-D uint8 tensor `buf` (CPU, ideally
    pinned); returns the number of bytes used."""
    import numpy as np
    view = buf.numpy()
    head = np.array([len(proofs)] + [len(p) for p in proofs], dtype="<u4").tobytes()
    blob = head + b"".join(proofs)
    if len(blob) > view.size:
        raise ValueError(f"proofs need {len(blob)} bytes, the gather buffer holds {view.size}")
    view[:len(blob)] = np.frombuffer(blob, dtype=np.uint8)
    return len(blob)


def unpack_proofs(buf):
    import numpy as np
    raw = buf.numpy()
    count = int(np.frombuffer(raw[:4].tobytes(), dtype="<u4")[0])
    lens = np.frombuffer(raw[4:4 + 4 * count].tobytes(), dtype="<u4")
    out, off = [], 4 + 4 * count
    for n in lens:
        out.append(raw[off:off + int(n)].tobytes())
        off += int(n)
    return out


class ProofGather:
    """Gathers every rank's list of proofs on rank 0 with one `dist.gather` of fixed-size byte
    tensors (device tensors with NCCL, CPU tensors with gloo); buffers are allocated once."""

    def __init__(self, dist, rank: int, world: int, cap_bytes: int, device=None):
        import torch
        self.dist, self.rank, self.world, self.device = dist, rank, world, device
        pin = device is not None
        self.host = torch.empty(cap_bytes, dtype=torch.uint8, pin_memory=pin)
        self.dev = torch.empty(cap_bytes, dtype=torch.uint8, device=device) if device is not None else None
        if rank == 0:
            self.all_host = [torch.empty(cap_bytes, dtype=torch.uint8, pin_memory=pin) for _ in range(world)]
            self.all_dev = [torch.empty(cap_bytes, dtype=torch.uint8, device=device) for _ in range(world)] if device is not None else None

    def gather(self, proofs):
        """Returns, on rank 0, the per-rank proof lists (index = rank); None elsewhere."""
        pack_proofs(proofs, self.host)
        if self.dev is not None:
            self.dev.copy_(self.host, non_blocking=True)
            self.dist.gather(self.dev, self.all_dev if self.rank == 0 else None, dst=0)
            if self.rank != 0:
                return None
            for h, d in zip(self.all_host, self.all_dev):
                h.copy_(d, non_blocking=True)
            import torch
            torch.cuda.current_stream().synchronize()
        else:
            self.dist.gather(self.host, self.all_host if self.rank == 0 else None, dst=0)
            if self.rank != 0:
                return None
        return [unpack_proofs(h) for h in self.all_host]
