"""Records what the reference's own NFS-store space manager does (compiled by oracle/Makefile from the
checkout: space_manager.cc, space_shard_layout.cc, space_shard_temp_layout.cc, file.cc, posix_file.cc)
for a fixed set of block ids and a fixed sequence of operations, into tests/golden/nfs_layout.json.

    python tests/golden/make_nfs_golden.py        # needs oracle/_ref (python -c "from oracle import oracle; oracle.build()")
"""
import hashlib
import json
import os
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle  # noqa: E402

BLOCK_SIZE = 1 << 16


def block_ids():
    ids = [b"0123456789abcdef", b"0123456789abcdef0123", bytes(range(16)), bytes(range(255, 223, -1))]
    for i in range(12):
        ids.append(hashlib.md5(b"block-%d" % i).hexdigest().encode())       # 32 hex characters, as UCM's hashes
    return ids


def listing(root):
    out = []
    for r, ds, fs in os.walk(root):
        rel = os.path.relpath(r, root)
        for f in fs:
            out.append([os.path.join(rel, f), os.path.getsize(os.path.join(r, f))])
        if not ds and not fs:
            out.append([rel + "/", -1])
    return sorted(out)


def scenario(mgr, ids):
    """A life cycle that touches every status the space manager can return."""
    trace = []
    a, b, c, d = ids[0], ids[2], ids[4], ids[5]
    trace.append(["new", a.hex(), mgr.new_block(a)])
    trace.append(["new", a.hex(), mgr.new_block(a)])              # in progress already
    trace.append(["lookup", a.hex(), int(mgr.lookup(a))])
    trace.append(["commit", a.hex(), mgr.commit(a, True)])
    trace.append(["lookup", a.hex(), int(mgr.lookup(a))])
    trace.append(["new", a.hex(), mgr.new_block(a)])              # committed already
    trace.append(["commit", b.hex(), mgr.commit(b, True)])        # never allocated
    trace.append(["new", c.hex(), mgr.new_block(c)])
    trace.append(["cancel", c.hex(), mgr.commit(c, False)])
    trace.append(["lookup", c.hex(), int(mgr.lookup(c))])
    trace.append(["new", c.hex(), mgr.new_block(c)])              # free again after the cancel
    trace.append(["new", d.hex(), mgr.new_block(d)])
    trace.append(["commit", d.hex(), mgr.commit(d, True)])
    return trace


def main():
    ids = block_ids()
    out = {"block_size": BLOCK_SIZE, "ids": [i.hex() for i in ids], "layouts": {}}
    for temp in (False, True):
        with tempfile.TemporaryDirectory() as d:
            mgr = oracle.RefSpaceManager(d, BLOCK_SIZE, temp)
            paths = [[os.path.relpath(mgr.path(i, True), d), os.path.relpath(mgr.path(i, False), d)] for i in ids]
            trace = scenario(mgr, ids)
            out["layouts"]["temp" if temp else "plain"] = {"paths": paths, "trace": trace, "listing": listing(d)}
    # which of three backends each id lands on
    with tempfile.TemporaryDirectory() as d:
        roots = [os.path.join(d, n) for n in ("b0", "b1", "b2")]
        for r in roots:
            os.makedirs(os.path.join(r, "data"))
        mgr = oracle.RefSpaceManager(":".join(roots), BLOCK_SIZE, False)
        out["backend_of"] = [int(os.path.relpath(mgr.path(i, False), d)[1]) for i in ids]
    with open(os.path.join(HERE, "nfs_layout.json"), "w") as f:
        json.dump(out, f, indent=1)
    print("wrote nfs_layout.json:", len(ids), "ids")


if __name__ == "__main__":
    main()
