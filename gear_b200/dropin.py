"""Register the mirrors under GEAR's own module names.

    import gear_b200.dropin; gear_b200.dropin.install()
    import gear, libgear.core as glibc          # now this build

Every submodule is aliased (not re-imported), so `gear.specs.ColumnSpec` and
`gear_b200.gear.specs.ColumnSpec` are the same object.
"""
import importlib
import pkgutil
import sys


def install(force: bool = False) -> None:
    for theirs, ours in (("libgear", "gear_b200.libgear"), ("gear", "gear_b200.gear")):
        if theirs in sys.modules and not force and not getattr(sys.modules[theirs], "__name__", "").startswith(ours):
            raise ImportError(f"a different '{theirs}' is already imported; pass force=True to replace it")
        pkg = importlib.import_module(ours)
        for m in pkgutil.walk_packages(pkg.__path__, ours + "."):
            importlib.import_module(m.name)
        for name, mod in list(sys.modules.items()):
            if name == ours or name.startswith(ours + "."):
                sys.modules[theirs + name[len(ours):]] = mod
