from .model import ExecDomain, MachineModel, Visibility, list_archs, load_machine

__all__ = ["ExecDomain", "MachineModel", "Visibility", "list_archs", "load_machine"]
