"""NVLink connectivity check (reference: stream_ep/utils.py:6-43).

Only boards whose name contains "PCIE" can lack NVLink between peers; SXM parts
(B200 HGX) are always fully connected through NVSwitch, so the check is skipped
for them exactly as in the reference.
"""
from __future__ import annotations

import os


def check_nvlink_connections(group) -> None:
    import torch

    if not torch.cuda.is_available():
        return
    name = torch.cuda.get_device_name()
    if "PCIE" not in name.upper():
        return
    try:
        import pynvml
    except ImportError:  # nvidia_ml_py missing: nothing to check with
        return
    import torch.distributed as dist

    pynvml.nvmlInit()
    try:
        devices = os.environ.get("CUDA_VISIBLE_DEVICES", "0,1,2,3,4,5,6,7").strip(",").split(",")
        physical = int(devices[torch.cuda.current_device()])
        size = group.size() if hasattr(group, "size") else group.Get_size()
        ids = [None] * size
        dist.all_gather_object(ids, physical, group)
        handles = [pynvml.nvmlDeviceGetHandleByIndex(i) for i in ids]
        for i, hi in enumerate(handles):
            for j, hj in enumerate(handles):
                if i >= j:
                    continue
                status = pynvml.nvmlDeviceGetP2PStatus(hi, hj, pynvml.NVML_P2P_CAPS_INDEX_NVLINK)
                assert status == pynvml.NVML_P2P_STATUS_OK, \
                    f"GPU {ids[i]} and GPU {ids[j]} are not connected through NVLink"
    finally:
        pynvml.nvmlShutdown()
