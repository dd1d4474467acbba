"""CPU oracle of the executor path (numpy).  Test infrastructure only: imported by tests/, `__graft_entry__.smoke()` and
bench.py's CPU-baseline legs, never by the kvm_b200 package."""
