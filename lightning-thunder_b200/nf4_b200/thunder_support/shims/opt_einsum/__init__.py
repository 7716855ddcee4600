"""Placeholder so that `import opt_einsum` succeeds; Thunder only needs it for einsum."""


def contract_path(*args, **kwargs):
    raise NotImplementedError("opt_einsum is not installed; einsum decomposition is unavailable")
