class _GlobalContext:
    """Single-process view: every group has size 1 and rank 0; no pipeline group."""
    _launched = False

    def get_local_rank(self, mode=None):
        return 0

    def get_world_size(self, mode=None):
        return 1

    def get_global_rank(self):
        return 0

    def is_initialized(self, mode=None):
        return False

    def get_group(self, mode=None):
        return None


global_context = _GlobalContext()
