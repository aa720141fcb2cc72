"""Multi-rank plumbing: the library-collective baseline layer; the symmetric-memory transport itself lives in
``streamep_b200.buffer`` (Python) and ``streamep_b200/csrc`` (native)."""
