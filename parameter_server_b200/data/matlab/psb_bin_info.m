function info = psb_bin_info(name)
% PSB_BIN_INFO  Parse name.info of a binary matrix into a struct:
%   type ('DENSE' | 'SPARSE' | 'SPARSE_BINARY'), row_major, rows, cols, nnz, sizeof_index, sizeof_value
% The file is protobuf text: "key: value" lines and "row { begin: B end: E }" / "col { ... }" ranges.
  txt = fileread([name '.info']);
  info = struct('type', 'SPARSE', 'row_major', true, 'rows', 0, 'cols', 0, 'nnz', 0, ...
                'sizeof_index', 8, 'sizeof_value', 4);
  tok = regexp(txt, 'type:\s*(\w+)', 'tokens', 'once');          if ~isempty(tok), info.type = tok{1}; end
  tok = regexp(txt, 'row_major:\s*(\w+)', 'tokens', 'once');     if ~isempty(tok), info.row_major = strcmp(tok{1}, 'true'); end
  tok = regexp(txt, 'nnz:\s*(\d+)', 'tokens', 'once');           if ~isempty(tok), info.nnz = str2double(tok{1}); end
  tok = regexp(txt, 'sizeof_index:\s*(\d+)', 'tokens', 'once');  if ~isempty(tok), info.sizeof_index = str2double(tok{1}); end
  tok = regexp(txt, 'sizeof_value:\s*(\d+)', 'tokens', 'once');  if ~isempty(tok), info.sizeof_value = str2double(tok{1}); end
  for which = {'row', 'col'}
    tok = regexp(txt, [which{1} '\s*\{[^}]*begin:\s*(\d+)[^}]*end:\s*(\d+)'], 'tokens', 'once');
    if ~isempty(tok)
      info.([which{1} 's']) = str2double(tok{2}) - str2double(tok{1});
    end
  end
end
