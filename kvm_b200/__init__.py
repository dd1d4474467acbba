"""B200-native executor for Magni VM task bundles: the persistent sm_100a kernel and the GPT op kernels behind the
reference's task ABI.  `kvm_b200.executor.Executor` is the host-side handle (ctypes over libkvm_b200.so)."""
__version__ = '0.1.0'
