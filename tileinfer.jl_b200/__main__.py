from tileinfer_b200.cli import main

main()
