"""TEST INFRASTRUCTURE, not product code: CPU restatements of the reference's path, used only
by tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs as the checker."""
