"""B200-native SquareQ weight streaming behind the Stagehand API (package under construction)."""
