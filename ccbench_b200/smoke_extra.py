"""Extra one-step checks run by smoke(); grows with the kernel families."""


def run() -> None:
    pass
