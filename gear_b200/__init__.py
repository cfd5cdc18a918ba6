"""gear_b200: B200-native replay sample + gather engine behind GEAR's interfaces.

    gear_b200.core      objects over the C ABI (table, handler, sampler, ...)
    gear_b200.sharded   trajectory-id sharded table + exchange
    gear_b200.libgear   mirror of GEAR's `libgear` pybind module
    gear_b200.gear      mirror of GEAR's `gear` Python package
    gear_b200.dropin    install() registers the two mirrors as `libgear` and `gear`
"""
__version__ = "0.1.0"
