"""Global switches, same names as torchsparse/backends.py:4-11.

``init`` is lazy about the device: importing the package must work on a machine
without a GPU (build and CPU-side tests run there)."""
import torch

benchmark = False
allow_tf32 = False
allow_fp16 = True
device_capability = 0
hash_rsv_ratio = 2  # table slots reserved per input point (>= 2)


def init():
    global benchmark, allow_tf32, allow_fp16, device_capability, hash_rsv_ratio
    benchmark = False
    if torch.cuda.is_available():
        cap = torch.cuda.get_device_capability()
        device_capability = cap[0] * 100 + cap[1] * 10
    else:
        device_capability = 0
    # fp32 inputs stay exact fp32 unless the user opts into TF32 (the reference turns TF32 on
    # for every Ampere-or-newer device, which silently changes fp32 results)
    allow_tf32 = False
    allow_fp16 = True
    hash_rsv_ratio = 2
