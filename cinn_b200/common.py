"""Types and targets, named as in the reference's `cinn.common` (cinn/pybind/common.cc)."""


class Type:
    def __init__(self, name):
        self.name = name

    def __repr__(self):
        return self.name

    def __eq__(self, other):
        return isinstance(other, Type) and other.name == self.name

    def __hash__(self):
        return hash(self.name)


def Float(bits):
    return Type({16: "float16", 32: "float32", 64: "float64"}[bits])


def Float16():
    return Type("float16")


def BFloat16():
    return Type("bfloat16")


def Int(bits):
    return Type({32: "int32", 64: "int64"}[bits])


def UInt(bits):
    return Type({8: "uint8"}[bits])


def Bool():
    return Type("bool")


class Target:
    """`arch` is "nvgpu" (device ordinal `device`) or "x86"."""

    def __init__(self, arch, device=0):
        self.arch = arch
        self.device = device

    def __repr__(self):
        return "Target(%s:%d)" % (self.arch, self.device)


def DefaultNVGPUTarget(device=0):
    return Target("nvgpu", device)


def DefaultHostTarget():
    """The reference's x86 target.  This library has no CPU execution path; compiling for it raises."""
    return Target("x86")


def DefaultTarget():
    return DefaultNVGPUTarget()
