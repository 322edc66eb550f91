"""Text and binary round trips: CSV, JSON, XML number lists and .npy (mirrors legacy/examples/tensor/demo_io_all.mojo)."""
import momijo.tensor as mt


def main():
    m = mt.from_list([[1.5, 2.0], [3.0, 4.0]])
    csv_text = mt.io.tensor_to_csv(m)
    json_text = mt.io.tensor_to_json_array(m)
    xml_text = mt.io.tensor_to_xml_numbers(m)
    assert mt.io.csv_to_tensor_with(csv_text).tolist() == m.tolist() == mt.io.json_numbers_to_tensor_with(json_text).tolist()
    assert mt.io.xml_numbers_to_tensor_with(xml_text).tolist() == m.tolist()
    mt.io.save_npy("m.npy", m)
    back = mt.io.load_npy("m.npy")
    assert mt.io.write_csv(m, None, "m.csv") and mt.io.read_csv_with("m.csv").tolist() == m.tolist()
    print(csv_text, json_text, xml_text, back.tolist(), sep="\n")
    assert back.tolist() == m.tolist()
    return back


if __name__ == "__main__":
    main()
