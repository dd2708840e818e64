from .group import CommError, Group, init_distributed, make_tp_pp_groups, shutdown_distributed

__all__ = ["CommError", "Group", "init_distributed", "make_tp_pp_groups", "shutdown_distributed"]
