"""ironpangu_b200 - a B200-native inference compiler and runtime.

Sub-packages: ``ops`` (sm_100a kernels behind a C ABI), ``parallel`` (symmetric heap and fused
collectives), ``models`` (model families on those kernels), ``runtime`` (engine, scheduler, server
bindings), ``compiler`` (DSL -> checked plan -> bundle, backed by the C++ core), ``utils``.
"""
__version__ = "0.1.0"
