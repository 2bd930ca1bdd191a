def write_all(ref):
    pass
