"""``import e3j_ops`` for the unmodified e3j Python: see `e3j_b200.e3j_ops_compat`."""

from e3j_b200.e3j_ops_compat import get_device_properties, get_kernel_registers, get_registrations  # noqa: F401
