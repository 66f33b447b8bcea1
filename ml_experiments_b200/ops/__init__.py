"""sm_100a operators (``torch.ops.b200``) and their Python / autograd wrappers."""
