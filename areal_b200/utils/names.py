"""Key layout of the name-resolve store (areal/utils/names.py)."""

import getpass

USER_NAMESPACE = getpass.getuser()


def _root(exp, trial):
    return f"{USER_NAMESPACE}/{exp}/{trial}"


def trial_root(exp, trial):
    return _root(exp, trial)


def gen_servers(exp, trial):
    return f"{_root(exp, trial)}/gen_servers"


def gen_server(exp, trial, idx):
    return f"{gen_servers(exp, trial)}/{idx}"


def update_weights_from_disk(exp, trial, version):
    return f"{_root(exp, trial)}/update_weights_from_disk/{version}"


def worker(exp, trial, role, idx):
    return f"{_root(exp, trial)}/workers/{role}/{idx}"


def workers(exp, trial, role):
    return f"{_root(exp, trial)}/workers/{role}"


def recover_flag(exp, trial):
    return f"{_root(exp, trial)}/recover"


def distributed_lock(exp, trial, name):
    return f"{_root(exp, trial)}/locks/{name}"


def registry_root(user: str | None = None):
    """Root under which every experiment of ``user`` registers (trial discovery across experiments)."""
    import getpass

    return f"registry/{user or getpass.getuser()}"


def trial_registry(exp, trial):
    """Record announcing that the trial exists (written by its launcher, listed by monitoring tools)."""
    import getpass

    return f"{registry_root(getpass.getuser())}/{exp}/{trial}"


def worker_discovery(exp, trial, role, idx="*"):
    """Key (or key prefix with ``idx="*"``) under which the workers of a role publish their addresses."""
    base = workers(exp, trial, role)
    return base if idx == "*" else worker(exp, trial, role, idx)
