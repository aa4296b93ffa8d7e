"""Multi-node search: tune/search.py reading the ``_ws{N}`` bandwidth file
(reference: tune/search_multinode.py)."""
import sys

import search

if __name__ == "__main__":
    sys.argv.append("--multinode")
    search.main()
