from chatlearn_b200.entrypoint import main

if __name__ == "__main__":
    main()
