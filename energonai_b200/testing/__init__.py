from .models import BoringModel, get_correct_output
