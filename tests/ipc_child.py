"""The engine's side of a cross-process registration (run by tests/test_gpu_ipc.py): reads pickled
IPC wrappers from a file, opens the parent's KV-cache memory, registers it, saves some blocks,
checks their host images against the bytes the parent expects, loads them into other block ids of
the parent's memory, and reports."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import pickle

    import pegaflow_b200 as pf
    from pegaflow_b200 import connector

    job = pickle.load(open(sys.argv[1], "rb"))
    eng = pf.PegaEngine(64 << 20, min_dma_bytes=64 << 10)
    client = connector.InProcEngineClient(eng)
    names = job["names"]
    ok, msg = client.register_context_batch(
        "ipc", "ns", 0, 0, 1, 1, job["device_id"], names, job["wrappers"], job["num_blocks"], job["bytes_per_block"],
        job["kv_stride_bytes"], job["segments"], "direct", False)
    assert ok, msg
    hashes = job["hashes"]
    saves = [(n, job["save_ids"], hashes) for n in names]
    ok, msg = client.save("ipc", 0, 0, job["device_id"], saves)
    assert ok, msg
    client.flush_saves()
    images_ok = True
    for li in range(len(names)):
        for j, h in enumerate(hashes):
            img = eng.block_slot_image("ipc", h, li)
            images_ok = images_ok and img is not None and [bytes(x) for x in img] == job["expected"][li][j]
    q = client.query_prefetch("ipc", hashes, "r")
    eng.batch_load("ipc", 0, job["device_id"], [names], [(q.lease, [job["load_ids"]])])
    m = eng.metrics()
    print(json.dumps({"images_ok": images_ok, "hits": q.num_hit_blocks, "load_failures": m["load_failures"],
                      "save_bytes": m["save_bytes"], "load_bytes": m["load_bytes"]}))
    sys.stdout.flush()
    eng.close()


if __name__ == "__main__":
    main()
