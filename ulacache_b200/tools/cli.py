"""``ulacache-kv-snapshot inspect|verify|commit <dir>`` and ``stripe <dir> --to <dir> --owners N`` (also
``python -m ulacache_b200.tools.cli``).  ``stripe`` converts a one-owner, one-request prefix snapshot into owner stripes.

Reference: ulacache/tools/cli.py:8-37.
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    from .snapshot.format import SnapshotReader, finalize_snapshot

    ap = argparse.ArgumentParser(prog="ulacache-kv-snapshot")
    ap.add_argument("command", choices=["inspect", "verify", "commit", "stripe"])
    ap.add_argument("path")
    ap.add_argument("--to", default="", help="stripe: the directory to create")
    ap.add_argument("--owners", type=int, default=0, help="stripe: number of owners")
    ap.add_argument("--chunk-rows", type=int, default=65536, help="stripe: rows of one plane held in memory at a time")
    args = ap.parse_args(argv)
    if args.command == "stripe":
        from .snapshot.prefix import stripe_prefix

        if not args.to or args.owners < 1:
            ap.error("stripe needs --to DIR and --owners N")
        commit = stripe_prefix(args.path, args.to, args.owners, chunk_rows=args.chunk_rows)
        print(json.dumps({"striped": True, "owners": len(commit["owners"]), "path": args.to}))
        return 0
    if args.command == "commit":
        commit = finalize_snapshot(args.path)
        print(json.dumps({"committed": True, "owners": len(commit["owners"]), "requests": commit["request_count"]}))
        return 0
    reader = SnapshotReader(args.path, require_committed=args.command == "verify", verify_payload=False)
    if args.command == "verify":
        print(json.dumps(reader.verify()))
        return 0
    lay = reader.layout
    print(json.dumps({"committed": reader.committed, "owners": lay.owners, "layers": lay.layers,
                      "kv_format": lay.kv_format, "mla_row_bytes": lay.mla_row_bytes,
                      "index_anchors": list(lay.index_anchors), "requests": len(reader.requests),
                      "tokens": sum(r.next_position for r in reader.requests)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
