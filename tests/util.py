"""Helpers shared by the GPU parity tests: storage-form numpy <-> device buffers with
guard zones (the reference harness' canary convention: fill byte 0xA5 around every
buffer, run_execution.py:75-85)."""
import numpy as np

GUARD = 4096
CANARY = 0xA5


def torch_dtype(dtype):
    import torch
    return {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[dtype]


def to_device(arr, dtype, device="cuda:0"):
    """storage-form numpy (float32 / float16 / uint16 bf16 bits) -> torch tensor on device."""
    import torch
    arr = np.ascontiguousarray(arr)
    if dtype == "bf16":
        return torch.from_numpy(arr.view(np.int16)).to(device).view(torch.bfloat16)
    return torch.from_numpy(arr).to(device)


def to_host(t, dtype):
    """torch tensor -> storage-form numpy."""
    import torch
    t = t.detach().cpu().contiguous()
    if dtype == "bf16":
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


class Guarded:
    """A device buffer with canary zones before and after the payload."""

    def __init__(self, shape, dtype, device="cuda:0", fill=None, offset=0):
        import torch
        self.dtype = dtype
        self.shape = tuple(shape)
        item = 4 if dtype == "fp32" else 2
        self.nbytes = int(np.prod(shape)) * item
        self.offset = GUARD + offset
        self.raw = torch.full((self.nbytes + 2 * GUARD + 256,), CANARY, dtype=torch.uint8, device=device)
        self.view = self.raw[self.offset:self.offset + self.nbytes].view(torch_dtype(dtype)).view(self.shape)
        if fill is not None:
            self.view.copy_(to_device(fill, dtype, device))

    def guards_intact(self):
        raw = self.raw.cpu().numpy()
        return bool((raw[:self.offset] == CANARY).all() and (raw[self.offset + self.nbytes:] == CANARY).all())

    def host(self):
        return to_host(self.view, self.dtype)
