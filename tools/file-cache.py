#!/usr/bin/env python3
"""
Command line access to the local file cache used by ``DistributeFilesDataset`` (``CachedFile``): copy files into the cache and
print the local paths, show what is cached, or clean up entries that were not used for a while.
(reference: tools/file-cache.py)
"""

import argparse
import os
import time
import _setup_returnn_env  # noqa: F401
from returnn_b200.utils.file_cache import FileCache


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("command", choices=["get", "list", "cleanup"])
    ap.add_argument("files", nargs="*")
    ap.add_argument("--cache-dir", default=None)
    ap.add_argument("--max-age-days", type=float, default=14.0)
    args = ap.parse_args()
    kwargs = {"cache_directory": args.cache_dir} if args.cache_dir else {}
    cache = FileCache(**kwargs)
    if args.command == "get":
        for fn in args.files:
            print(cache.get_file(os.path.abspath(fn)))
    elif args.command == "list":
        root = cache.cache_directory
        for dirpath, _, names in os.walk(root):
            for n in names:
                p = os.path.join(dirpath, n)
                print("%10i  %s  %s" % (os.path.getsize(p), time.strftime("%Y-%m-%d %H:%M", time.localtime(os.path.getatime(p))), p))
    else:
        limit = time.time() - args.max_age_days * 86400
        removed = 0
        for dirpath, _, names in os.walk(cache.cache_directory):
            for n in names:
                p = os.path.join(dirpath, n)
                if os.path.getatime(p) < limit:
                    os.remove(p)
                    removed += 1
        print("removed %i files" % removed)


if __name__ == "__main__":
    main()
