import socket

import torch


def get_current_device():
    return torch.device("cpu")


def is_using_pp():
    return False


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]
