"""Instance B of a cross-process prefix hit (run by tests/test_gpu_peer.py): opens the KV-cache regions
another process exported, pulls some blocks of every layer into its own cache on another GPU with the
peer-copy kernel, and compares its whole cache with what the owner's seed says it must hold."""
import ctypes as C
import json
import os
import pickle
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import numpy as np
    import torch

    import pegaflow_b200 as pf
    from pegaflow_b200 import _native as N

    job = pickle.load(open(sys.argv[1], "rb"))
    dst_dev, nb, seg, L = job["dst_device"], job["num_blocks"], job["seg"], len(job["regions"])
    torch.cuda.set_device(dst_dev)
    device = torch.device("cuda", dst_dev)
    regions = [N.IpcRegion.from_buffer_copy(b) for b in job["regions"]]
    ptrs, src_dev = [], None
    for r in regions:
        ptr, dev = C.c_uint64(), C.c_int()
        N.check(N.lib.pf_ipc_open_for(C.byref(r), dst_dev, C.byref(ptr), C.byref(dev)))
        ptrs.append(ptr.value)
        src_dev = dev.value
    dst = [torch.zeros((2, nb, seg), dtype=torch.uint8, device=device) for _ in range(L)]
    be = pf.TransferBackend(dst_dev)
    stream = torch.cuda.Stream()
    sids, dids = np.asarray(job["src_ids"], dtype=np.uint32), np.asarray(job["dst_ids"], dtype=np.uint32)
    be.peer_copy_layers([(p, seg, nb * seg, seg, 2, nb) for p in ptrs], sids,
                        [(t.data_ptr(), seg, nb * seg, seg, 2, nb) for t in dst], dids, stream.cuda_stream)
    stream.synchronize()
    ok = True
    for l, t in enumerate(dst):
        src = np.random.default_rng(job["seed"] + l).integers(0, 256, size=(2, nb, seg), dtype=np.uint8)
        want = np.zeros((2, nb, seg), dtype=np.uint8)
        want[:, dids.astype(np.int64)] = src[:, sids.astype(np.int64)]
        ok = ok and np.array_equal(t.cpu().numpy(), want)
    st = be.stats()
    be.close()
    for r in regions:
        N.check(N.lib.pf_ipc_close_for(C.byref(r), dst_dev))
    print(json.dumps({"bit_exact": bool(ok), "src_device": src_dev, "bytes_peer": st["bytes_peer"],
                      "device_status": st["device_status"], "kernel_launches": st["kernel_launches"]}))
    sys.stdout.flush()


if __name__ == "__main__":
    main()
